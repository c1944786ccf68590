"""Host-side mirror of dlf's tensor front-end for the dense-contraction path.

``gemm`` / ``matmul`` / ``dot`` / ``conv2d`` follow dlf/include/tensor/linalg.h:42-101, 339-450,
511-549 and dlf/include/tensor/dnn.h:186-201 for *device* tensors: they derive leading
dimensions and transposes from strides, broadcast batch prefixes, reorder operands BLAS cannot
express, and route to ``gblas.gemm`` / ``gblas.gemmStridedBatched`` / ``gblas.gemmBatched`` /
``gdnn.conv2d`` exactly where ``detail::matmul`` for ``gpgpu::Buffer<T>`` does
(dlf/include/tensor/linalg_detail.h:1573-1662). A device tensor is a torch CUDA tensor (any
strides / storage offset). The routines never compute on the host; the ``backend`` argument exists
so the routing can be exercised against another implementation of the same four routines.
"""
import torch

from . import gblas as _gblas
from . import gdnn as _gdnn
from .gblas import Layout, Transpose


class ShapeError(ValueError):
    """Counterpart of dlf's shape_error."""


def _flat(t):
    """The tensor's whole storage as a flat buffer (the reference's Buffer<T>)."""
    n = t.untyped_storage().nbytes() // t.element_size()
    return torch.empty(0, dtype=t.dtype, device=t.device).set_(t.untyped_storage(), 0, (n,), (1,))


def gemm(transA, transB, alpha, A, B, beta, C, Y=None, backend=None):
    """Y = alpha*op(A)*op(B) + beta*broadcast(C)  (dlf::gemm, linalg.h:42-101).

    A, B are 2-D row-major device tensors whose rows may be padded (ld = stride(0)); C is
    broadcast to {m, n}. Returns Y (allocated when not given)."""
    be = backend or _gblas
    if A.dim() != 2 or B.dim() != 2:
        raise ShapeError("gemm: A and B must be matrices")
    if A.stride(1) != 1 or B.stride(1) != 1:
        raise ShapeError("gemm: rows of A and B must be contiguous")
    m, k = A.shape
    if transA != Transpose.NoTrans:
        m, k = k, m
    p, n = B.shape
    if transB != Transpose.NoTrans:
        p, n = n, p
    if k != p:
        raise ShapeError("gemm: incompatible shape")
    if Y is None:
        Y = torch.empty((m, n), dtype=A.dtype, device=A.device)
    elif tuple(Y.shape) != (m, n) or Y.stride(1) != 1:
        raise ShapeError("gemm: bad output shape")
    if beta != 0:
        try:
            Y.copy_(C.expand(m, n))
        except RuntimeError:
            raise ShapeError("gemm: C is not broadcastable to {m, n}")
    be.gemm(Layout.RowMajor, transA, transB, m, n, k, alpha,
            _flat(A), A.storage_offset(), max(A.stride(0), 1),
            _flat(B), B.storage_offset(), max(B.stride(0), 1), beta,
            _flat(Y), Y.storage_offset(), max(Y.stride(0), 1))
    return Y


def _is_contiguous_strides(shape, strides):
    """is_contiguous_strides (linalg_detail.h:1391-1410): batch dims collapse to one stride."""
    r = len(shape)
    if r <= 2:
        return True
    s = strides[r - 3]
    if s == 0:
        return all(strides[i] == 0 for i in range(r - 4, -1, -1))
    for i in range(r - 4, -1, -1):
        if strides[i] != s * shape[i]:
            return False
        s = strides[i]
    return True


def _lhs_need_reorder(m, n, k, lda, incA):
    """is_matmul_lhs_need_reorder for GPU tensors (linalg_detail.h:1412-1432)."""
    if lda == 0 or incA == 0:
        return True
    if lda < 0 or incA < 0:
        return True
    if m == 1 and n == 1:
        return False
    if lda != 1 and incA != 1:
        return True
    if incA == 1 and lda < k:
        return True
    if lda == 1 and incA < m:
        return True
    return False


def _rhs_need_reorder(k, n, ldb, incB):
    """is_matmul_rhs_need_reorder for GPU tensors (linalg_detail.h:1434-1454)."""
    if ldb == 0 or incB == 0:
        return True
    if ldb < 0 or incB < 0:
        return True
    if n == 1:
        return False
    if ldb != 1 and incB != 1:
        return True
    if incB == 1 and ldb < n:
        return True
    if ldb == 1 and incB < k:
        return True
    return False


def _broadcast(A, B):
    """matmul_broadcast (linalg_detail.h:1342-1389) on torch views; returns (A, B, shapeC, batch)."""
    if A.dim() == 0 or B.dim() == 0:
        raise ShapeError("matmul: Input tensors of wrong rank (0).")
    if A.dim() == 1:
        A = A.unsqueeze(0)
    if B.dim() == 1:
        B = B.unsqueeze(1)
    m, k = A.shape[-2:]
    p, n = B.shape[-2:]
    if k != p:
        raise ShapeError("matmul: Incompatible dimensions for matrix multiplication")
    try:
        prefix = torch.broadcast_shapes(tuple(A.shape[:-2]), tuple(B.shape[:-2]))
    except RuntimeError:
        raise ShapeError("matmul: batch dimensions are not broadcastable")
    A = A.expand(*prefix, m, k)
    B = B.expand(*prefix, k, n)
    batch = 1
    for e in prefix:
        batch *= e
    return A, B, tuple(prefix) + (m, n), batch


def _linear_offset(shape, strides, offset, index):
    """Shape::linear_offset: storage offset of the element with row-major linear index."""
    off = offset
    for extent, stride in zip(reversed(shape), reversed(strides)):
        off += (index % extent) * stride
        index //= extent
    return off


def matmul(A, B, C=None, alpha=1, beta=0, backend=None, trace=None):
    """C = alpha * A @ B + beta * C with numpy-style batch broadcasting (dlf::matmul,
    linalg.h:339-450). ``trace`` (a list) receives the name of the routine the call was routed
    to, which is how the tests pin the routing of detail::matmul."""
    be = backend or _gblas
    a_vec, b_vec = A.dim() == 1, B.dim() == 1
    vA, vB, shapeC, batch = _broadcast(A, B)
    m, k = vA.shape[-2:]
    n = vB.shape[-1]
    lda, incA = vA.stride(-2), vA.stride(-1)
    ldb, incB = vB.stride(-2), vB.stride(-1)
    if lda == 0 and m == 1:
        lda = k
    if ldb == 0 and k == 1:
        ldb = n
    if incA == 0 and k == 1:
        incA = 1
    if incB == 0 and n == 1:
        incB = 1

    # torch reports arbitrary strides for size-1 dims; BLAS only needs them to be legal
    if m == 1 and incA == 1:
        lda = max(lda, k)
    if k == 1 and incB == 1:
        ldb = max(ldb, n)

    if _lhs_need_reorder(m, n, k, lda, incA):
        tmp = A.contiguous()
        vA, _, _, _ = _broadcast(tmp, B)
        lda, incA = k, 1
    if _rhs_need_reorder(k, n, ldb, incB):
        tmp = B.contiguous()
        _, vB, _, _ = _broadcast(A, tmp)
        ldb, incB = n, 1

    out_shape = list(shapeC)
    if a_vec:
        del out_shape[-2]
    if b_vec:
        del out_shape[-1]
    if C is None:
        if beta != 0:
            raise ShapeError("matmul: beta != 0 needs an output tensor")
        C = torch.empty(out_shape, dtype=A.dtype, device=A.device)
    elif list(C.shape) != out_shape:
        raise ShapeError("matmul: bad output shape")
    vC = C
    if b_vec:
        vC = vC.unsqueeze(-1)
    if a_vec:
        vC = vC.unsqueeze(-2)
    ldc, incC = vC.stride(-2), vC.stride(-1)
    if (ldc == 0 or m == 1) and incC == 1:
        ldc = max(ldc, n)
    if n == 1:
        incC = 1
        ldc = max(ldc, 1)
    if incC != 1 or ldc < n:
        raise ShapeError("matmul: the output tensor must be contiguous")

    transA = Transpose.NoTrans
    if incA != 1:
        transA, lda = Transpose.Trans, incA
    transB = Transpose.NoTrans
    if incB != 1:
        transB, ldb = Transpose.Trans, incB
    # a 1 x k (or k x 1) operand seen as transposed still needs a legal leading dimension
    if transA == Transpose.Trans:
        lda = max(lda, m)
    if transB == Transpose.Trans:
        ldb = max(ldb, k)

    fa, fb, fc = _flat(vA), _flat(vB), _flat(vC)
    sa, sb, sc = list(vA.stride()), list(vB.stride()), list(vC.stride())
    if batch == 1:
        # the reference sends m == n == 1 to gblas::dot and n == 1 to gblas::gemv; both are the
        # same contraction, served here by the gemm entry point
        if trace is not None:
            trace.append("gemm")
        be.gemm(Layout.RowMajor, transA, transB, m, n, k, alpha, fa, vA.storage_offset(), lda,
                fb, vB.storage_offset(), ldb, beta, fc, vC.storage_offset(), ldc)
    elif (_is_contiguous_strides(vA.shape, sa) and _is_contiguous_strides(vB.shape, sb) and
          _is_contiguous_strides(vC.shape, sc)):
        if trace is not None:
            trace.append("gemmStridedBatched")
        be.gemmStridedBatched(Layout.RowMajor, transA, transB, m, n, k, alpha,
                              fa, vA.storage_offset(), lda, sa[-3],
                              fb, vB.storage_offset(), ldb, sb[-3], beta,
                              fc, vC.storage_offset(), ldc, sc[-3], batch)
    else:
        if trace is not None:
            trace.append("gemmBatched")
        a_off = [_linear_offset(vA.shape, sa, vA.storage_offset(), p * m * k) for p in range(batch)]
        b_off = [_linear_offset(vB.shape, sb, vB.storage_offset(), p * k * n) for p in range(batch)]
        c_off = [_linear_offset(vC.shape, sc, vC.storage_offset(), p * m * n) for p in range(batch)]
        be.gemmBatched(Layout.RowMajor, transA, transB, m, n, k, [alpha] * batch, fa, a_off, lda,
                       fb, b_off, ldb, [beta] * batch, fc, c_off, ldc, batch)
    return C


def dot(A, B, backend=None):
    """dlf::dot (linalg.h:511-549): scalars scale, everything else is matmul after the N-D
    operand's contraction axis is brought to matmul's convention."""
    if A.dim() == 0 or B.dim() == 0:
        return A * B
    if A.dim() <= 2 and B.dim() <= 2:
        return matmul(A, B, backend=backend)
    # N-D: sum over the last axis of A and the second-to-last of B
    if B.dim() == 1:
        return matmul(A, B, backend=backend)
    a_shape, b_shape = list(A.shape), list(B.shape)
    A2 = A.reshape(-1, a_shape[-1]) if A.is_contiguous() else A.contiguous().reshape(-1, a_shape[-1])
    Bm = B.movedim(-2, 0).reshape(b_shape[-2], -1)
    out = matmul(A2, Bm.contiguous() if not Bm.is_contiguous() else Bm, backend=backend)
    return out.reshape(a_shape[:-1] + b_shape[:-2] + b_shape[-1:])


def symm(side, uplo, A, B, alpha=1, beta=0, C=None, backend=None):
    """dlf::symm (linalg.h:132-163): C = alpha*S*B + beta*C (Left) or alpha*B*S + beta*C (Right) for
    2-D tensors; S is the symmetric matrix whose `uplo` triangle is the leading block of A."""
    be = backend or _gblas
    if A.dim() != 2 or B.dim() != 2:
        raise ShapeError("symm: matrices expected")
    m, n = B.shape
    k = m if int(side) == _gblas.Side.Left else n
    if A.shape[0] < k or A.shape[1] < k:
        raise ShapeError("symm: matrix A has too few dimensions")
    if not (A.stride(1) == 1 and B.is_contiguous()):
        raise ShapeError("symm: operands must be row-major")
    if C is None:
        if beta != 0:
            raise ShapeError("symm: beta != 0 needs an output tensor")
        C = torch.empty((m, n), dtype=A.dtype, device=A.device)
    elif tuple(C.shape) != (m, n) or not C.is_contiguous():
        raise ShapeError("symm: bad output tensor")
    be.symm(Layout.RowMajor, side, uplo, m, n, alpha, _flat(A), A.storage_offset(), A.stride(0), _flat(B),
            B.storage_offset(), B.stride(0), beta, _flat(C), C.storage_offset(), C.stride(0))
    return C


def _triangular(name, side, uplo, transA, diag, A, B, alpha, backend):
    be = backend or _gblas
    if A.dim() != 2 or B.dim() != 2:
        raise ShapeError(name + ": matrices expected")
    m, n = B.shape
    k = m if int(side) == _gblas.Side.Left else n
    if A.shape[0] < k or A.shape[1] < k:
        raise ShapeError(name + ": matrix A has too few dimensions")
    if A.stride(1) != 1:
        raise ShapeError(name + ": A must be row-major")
    C = B.contiguous().clone()  # the reference copies B into the result and works in place (linalg.h:252-258)
    getattr(be, name)(Layout.RowMajor, side, uplo, transA, diag, m, n, alpha, _flat(A), A.storage_offset(),
                      A.stride(0), _flat(C), C.storage_offset(), C.stride(0))
    return C


def trmm(side, uplo, transA, diag, A, B, alpha=1, backend=None):
    """dlf::trmm (linalg.h:240-276): alpha*op(T)*B (Left) or alpha*B*op(T) (Right) as a new tensor."""
    return _triangular("trmm", side, uplo, transA, diag, A, B, alpha, backend)


def trsm(side, uplo, transA, diag, A, B, alpha=1, backend=None):
    """dlf::trsm (linalg.h:278-314): the solution X of op(T)*X = alpha*B (Left) or X*op(T) = alpha*B."""
    return _triangular("trsm", side, uplo, transA, diag, A, B, alpha, backend)


def _matrix_chain_order(dims):
    """detail::matrix_chain_order (linalg_detail.h:1701-1720): split table of the cheapest
    parenthesisation of a chain whose i-th matrix is dims[i] x dims[i+1]."""
    n = len(dims) - 1
    inf = float("inf")
    cost = [[0 if i == j else inf for j in range(n)] for i in range(n)]
    split = [[0] * n for _ in range(n)]
    for length in range(1, n):
        for i in range(n - length):
            j = i + length
            for k in range(i, j):
                c = cost[i][k] + cost[k + 1][j] + dims[i] * dims[k + 1] * dims[j + 1]
                if c < cost[i][j]:
                    cost[i][j] = c
                    split[i][j] = k
    return split


def multi_dot(*args, backend=None):
    """dlf::multi_dot (linalg.h:569-603): the product of a chain of matrices, evaluated in the
    order that costs the fewest multiplications. A 1-D first argument is a row vector, a 1-D last
    argument a column vector, everything in between must be 2-D (linalg_detail.h:1664-1699)."""
    if len(args) == 1 and isinstance(args[0], (list, tuple)):
        args = tuple(args[0])
    if len(args) == 0:
        raise ValueError("multi_dot: at least 1 argument is required")
    if len(args) == 1:
        return args[0]
    first = args[0]
    if first.dim() == 1:
        dims = [1, first.shape[0]]
    elif first.dim() == 2:
        dims = [first.shape[0], first.shape[1]]
    else:
        raise ShapeError("multi_dot: the first argument must be a vector or a matrix")
    n = dims[1]
    for i, t in enumerate(args[1:], start=1):
        if t.dim() == 2:
            if t.shape[0] != n:
                raise ShapeError("multi_dot: incompatible shape")
            n = t.shape[1]
        elif i == len(args) - 1 and t.dim() == 1:
            if t.shape[0] != n:
                raise ShapeError("multi_dot: incompatible shape")
            n = 1
        else:
            raise ShapeError("multi_dot: the arguments in the middle must be matrices")
        dims.append(n)
    split = _matrix_chain_order(dims)

    def product(i, j):
        if i == j:
            return args[i]
        return matmul(product(i, split[i][j]), product(split[i][j] + 1, j), backend=backend)

    return product(0, len(args) - 1)


def conv2d(X, W, Y, filt, bias=None, backend=None):
    """dlf::dnn::conv2d(X, W, Y, filter) (dnn.h:186-201) for contiguous NCHW / OIHW device tensors,
    with the optional bias of ConvOp (predict.h:1272-1281) fused in."""
    be = backend or _gdnn
    if tuple(X.shape) != (filt.batches, filt.channels, filt.height, filt.width):
        raise ShapeError("conv2d: input shape does not match the filter")
    if tuple(W.shape) != (filt.num_kernels, filt.channels // filt.group, filt.kernel_h,
                          filt.kernel_w):
        raise ShapeError("conv2d: kernel shape does not match the filter")
    if not (X.is_contiguous() and W.is_contiguous()):
        raise ShapeError("conv2d: X and W must be contiguous")
    if Y is None:
        Y = torch.empty(filt.output_shape(), dtype=X.dtype, device=X.device)
    elif tuple(Y.shape) != tuple(filt.output_shape()) or not Y.is_contiguous():
        raise ShapeError("conv2d: bad output tensor")
    be.conv2d_filter(X, W, Y, filt, bias=bias)
    return Y
