"""Shared helpers of the test-suite: golden-fixture decoding, a tiny evaluator for the tensor
expressions that appear in the reference's matmul tests, and the oracle-backed stand-in for the
gblas routines used to exercise the front-end routing on CPU tensors."""
import json
import os
import re

import numpy as np
import torch

import oracle

HERE = os.path.dirname(os.path.abspath(__file__))


def load_goldens():
    with open(os.path.join(HERE, "golden", "reference_goldens.json")) as f:
        return json.load(f)


def tensor_of(spec, dtype=torch.float32):
    shape = spec["shape"]
    n = int(np.prod(shape)) if shape else 1
    if "range" in spec:
        t = torch.arange(spec["range"], spec["range"] + n, dtype=torch.float64)
    elif "fill" in spec:
        t = torch.full((n,), float(spec["fill"]), dtype=torch.float64)
    else:
        t = torch.tensor(spec["values"], dtype=torch.float64)
    return t.to(dtype).reshape(shape)


def _slice(t, spec):
    idx = []
    for part in spec.split(","):
        part = part.strip()
        if ":" in part:
            f = [int(x) if x.strip() else None for x in part.split(":")]
            idx.append(slice(*f))
        else:
            # dlf keeps an integer-indexed axis as an extent-1 axis in string slices
            i = int(part)
            idx.append(slice(i, i + 1 if i != -1 else None))
    if any(isinstance(i, slice) and i.step is not None and i.step < 0 for i in idx):
        # torch has no negative strides; the reference reorders such operands on the GPU anyway
        return torch.from_numpy(np.ascontiguousarray(t.cpu().numpy()[tuple(idx)])).to(t.device)
    return t[tuple(idx)]


def evaluate(expr, env):
    """Evaluates one of the tensor expressions used by MatMulTest against `env` (name -> spec)."""
    expr = expr.strip()
    m = re.fullmatch(r"flip\((.*)\)", expr)
    if m:
        t = evaluate(m.group(1), env)
        return torch.flip(t, dims=[t.dim() - 1]).contiguous()
    m = re.fullmatch(r"unsqueeze\((\w+),\s*([\d,\s]+)\)", expr)
    if m:
        t = evaluate(m.group(1), env)
        for ax in [int(x) for x in m.group(2).split(",")]:
            t = t.unsqueeze(ax)
        return t
    m = re.fullmatch(r"as_strided\((\w+),\s*\{([^}]*)\},\s*\{([^}]*)\}\)", expr)
    if m:
        t = evaluate(m.group(1), env)
        return torch.as_strided(t, [int(x) for x in m.group(2).split(",")],
                                [int(x) for x in m.group(3).split(",")])
    m = re.fullmatch(r"(\w+)\.transpose\(([\d,\s]*)\)", expr)
    if m:
        t = evaluate(m.group(1), env)
        perm = [int(x) for x in m.group(2).split(",")] if m.group(2).strip() else \
            list(range(t.dim() - 1, -1, -1))
        return t.permute(perm)
    m = re.fullmatch(r"(\w+)\.broadcast_to\(\{([^}]*)\}\)", expr)
    if m:
        return evaluate(m.group(1), env).expand([int(x) for x in m.group(2).split(",")])
    m = re.fullmatch(r'(\w+)\["([^"]*)"\]', expr)
    if m:
        return _slice(evaluate(m.group(1), env), m.group(2))
    m = re.fullmatch(r"(\w+)\[(\d+)\]", expr)
    if m:
        return evaluate(m.group(1), env)[int(m.group(2))]
    if re.fullmatch(r"\w+", expr):
        spec = env[expr]
        if isinstance(spec, torch.Tensor):
            return spec
        if "expr" in spec:
            return evaluate(spec["expr"], env)
        return tensor_of(spec, env.get("__dtype__", torch.float32))
    raise NotImplementedError(expr)


UNSUPPORTED_EXPR = ("partition(",)


class OracleBlas:
    """The three gblas routines served by the CPU oracle on flat CPU torch buffers (float32, or
    int32 through the reference's generic gemm). Lets tensor.matmul's routing run without a GPU."""

    def __init__(self):
        self.calls = []

    @staticmethod
    def _np(buf):
        return buf.numpy()

    def gemm(self, layout, ta, tb, m, n, k, alpha, a, a_off, a_ld, b, b_off, b_ld, beta, c, c_off,
             c_ld, queue=None, event=None):
        self.calls.append("gemm")
        if c.dtype == torch.float32:
            oracle.gblas_sgemm(int(layout), int(ta), int(tb), m, n, k, float(alpha), self._np(a),
                               a_off, a_ld, self._np(b), b_off, b_ld, float(beta), self._np(c),
                               c_off, c_ld)
        else:
            assert int(layout) == oracle.ROW_MAJOR
            oracle.gemm_generic(int(ta), int(tb), m, n, k, int(alpha), self._np(a)[a_off:], a_ld,
                                self._np(b)[b_off:], b_ld, int(beta), self._np(c)[c_off:], c_ld)

    def gemmStridedBatched(self, layout, ta, tb, m, n, k, alpha, a, a_off, a_ld, a_st, b, b_off,
                           b_ld, b_st, beta, c, c_off, c_ld, c_st, batch, queue=None, event=None):
        self.calls.append("gemmStridedBatched")
        for i in range(batch):
            self.gemm(layout, ta, tb, m, n, k, alpha, a, a_off + i * a_st, a_ld, b,
                      b_off + i * b_st, b_ld, beta, c, c_off + i * c_st, c_ld)
            self.calls.pop()

    def gemmBatched(self, layout, ta, tb, m, n, k, alphas, a, a_offs, a_ld, b, b_offs, b_ld, betas,
                    c, c_offs, c_ld, batch, queue=None, event=None):
        self.calls.append("gemmBatched")
        for i in range(batch):
            self.gemm(layout, ta, tb, m, n, k, alphas[i], a, a_offs[i], a_ld, b, b_offs[i], b_ld,
                      betas[i], c, c_offs[i], c_ld)
            self.calls.pop()


def rel_fro(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-300))


def max_rel(got, ref, eps=1e-2):
    """max |x-y| / max(|y|, eps*max|y|): the fp16/bf16 parity metric (eps keeps near-zero
    outputs from dominating)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.maximum(np.abs(ref), eps * np.abs(ref).max())
    return float((np.abs(got - ref) / den).max())
