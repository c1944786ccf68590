"""Sharding of the hot path over the GPUs of one box: one process per GPU, torch.distributed
for the plumbing (NCCL on GPUs; the same code runs over gloo in the CPU tests).

The reference has no collectives at all: its multi-GPU story is one device per host thread
(gpgpu/src/gpgpu.cpp:139-168). The path shards naturally:

* conv2d and batched GEMM: images / batch entries are independent, so each rank takes a
  contiguous slab (``split``) and nothing is exchanged on the data path;
* one large GEMM: rank r computes a block of rows of C (``gemm_row_sharded``); the only exchange
  is an all-gather of those row blocks so that every rank ends with the whole C.
"""
import torch
import torch.distributed as dist

from . import gblas as _gblas
from .gblas import Layout, Transpose
from .tensor import ShapeError, _flat


def split(total, world, rank):
    """Contiguous partition of range(total): returns (start, count) of `rank`'s slab. The first
    ``total % world`` ranks get one extra unit."""
    base, extra = divmod(int(total), int(world))
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def all_gather_rows(C, world, rank, group=None):
    """Every rank holds valid rows split(M, world, rank) of the row-major 2-D tensor C; afterwards
    every rank holds all rows. Equal slabs use one in-place all-gather, ragged ones a broadcast
    per owner."""
    if world == 1:
        return C
    M = C.shape[0]
    if not C.is_contiguous():
        raise ShapeError("all_gather_rows: C must be contiguous")
    if M % world == 0:
        start, cnt = split(M, world, rank)
        dist.all_gather_into_tensor(C.view(-1), C[start:start + cnt].reshape(-1), group=group)
    else:
        for r in range(world):
            s, c = split(M, world, r)
            if c:
                dist.broadcast(C[s:s + c], src=r, group=group)
    return C


_COMM_STREAMS = {}


def _comm_stream(device):
    s = _COMM_STREAMS.get(device.index)
    if s is None:
        s = torch.cuda.Stream(device=device)
        _COMM_STREAMS[device.index] = s
    return s


def gemm_row_sharded_overlapped(transA, transB, alpha, A, B, beta, C, world, rank, panels, group=None,
                                backend=None):
    """As gemm_row_sharded, with the exchange hidden behind the arithmetic: the rows of C are cut
    into `panels` panels, every rank computes its 1/world slice of each panel in turn, and the
    all-gather of a finished panel (in place: a panel is one contiguous block of C and the
    rank's slice lies inside it) runs on a second stream while the next panel is computed.
    Needs m divisible by world * panels; the result is the same C on every rank."""
    be = backend or _gblas
    m, k = (A.shape[0], A.shape[1]) if transA == Transpose.NoTrans else (A.shape[1], A.shape[0])
    n = B.shape[1] if transB == Transpose.NoTrans else B.shape[0]
    if tuple(C.shape) != (m, n) or not C.is_contiguous():
        raise ShapeError("gemm_row_sharded_overlapped: bad output")
    if panels < 1 or m % (world * panels) != 0:
        raise ShapeError("gemm_row_sharded_overlapped: m must be divisible by world * panels")
    rows_p, rows_s = m // panels, m // (panels * world)
    cuda = C.is_cuda
    cur = torch.cuda.current_stream(C.device) if cuda else None
    comm = _comm_stream(C.device) if cuda and world > 1 else None
    for pnl in range(panels):
        r0 = pnl * rows_p + rank * rows_s
        a_off = A.storage_offset() + (r0 * A.stride(0) if transA == Transpose.NoTrans else r0)
        be.gemm(Layout.RowMajor, transA, transB, rows_s, n, k, alpha, _flat(A), a_off, A.stride(0),
                _flat(B), B.storage_offset(), B.stride(0), beta, _flat(C),
                C.storage_offset() + r0 * C.stride(0), C.stride(0))
        if world == 1:
            continue
        panel = C[pnl * rows_p:(pnl + 1) * rows_p].view(-1)
        mine = C[r0:r0 + rows_s].reshape(-1)
        if comm is not None:
            comm.wait_event(cur.record_event())
            with torch.cuda.stream(comm):
                dist.all_gather_into_tensor(panel, mine, group=group)
        else:
            dist.all_gather_into_tensor(panel, mine, group=group)
    if comm is not None:
        cur.wait_stream(comm)
    return C


def gemm_row_sharded(transA, transB, alpha, A, B, beta, C, world, rank, group=None, backend=None,
                     gather=True):
    """C = alpha*op(A)*op(B) + beta*C (row-major, all operands replicated on every rank) with the
    rows of C partitioned over the ranks, then all-gathered. A row block of op(A) is a row slab of
    A when A is not transposed and a column slab of the stored k x m matrix when it is: either way
    it is the same buffer with an element offset and the unchanged leading dimension, so nothing
    is copied."""
    be = backend or _gblas
    if A.dim() != 2 or B.dim() != 2 or C.dim() != 2:
        raise ShapeError("gemm_row_sharded: matrices expected")
    m, k = (A.shape[0], A.shape[1]) if transA == Transpose.NoTrans else (A.shape[1], A.shape[0])
    n = B.shape[1] if transB == Transpose.NoTrans else B.shape[0]
    if tuple(C.shape) != (m, n):
        raise ShapeError("gemm_row_sharded: bad output shape")
    r0, cnt = split(m, world, rank)
    if cnt:
        a_off = A.storage_offset() + (r0 * A.stride(0) if transA == Transpose.NoTrans else r0)
        be.gemm(Layout.RowMajor, transA, transB, cnt, n, k, alpha, _flat(A), a_off, A.stride(0),
                _flat(B), B.storage_offset(), B.stride(0), beta, _flat(C),
                C.storage_offset() + r0 * C.stride(0), C.stride(0))
    if gather:
        all_gather_rows(C, world, rank, group)
    return C
