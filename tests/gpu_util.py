"""numpy-in / numpy-out helpers around the cuda backend for the GPU parity tests."""
from __future__ import annotations

import numpy as np

from halo_b200 import backend as hb
from halo_b200 import synth


class Harness:
    def __init__(self, device: int = 0):
        self.be = hb.CudaBackend(device)
        self.st = self.be.create_stream()

    def gemv(self, wtype, w, x, rows, cols, *, variant=0, allow_gemm=False, w_stride=0, w_offset=0, x_stride=0, y_stride=0,
             y_guard=0):
        """Runs Backend::gemv on host arrays; y is returned as [n_vec, rows].  With y_guard > 0 the output buffer is
        padded with sentinel floats on both sides and the sentinels are checked (the reference's "y padding must
        survive" check, tests/unit/hip/test_hip_gemv.cpp:200-205)."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
        n_vec = x.shape[0]
        wb = self.be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
        xs = x_stride or cols * 4
        xbuf = np.zeros(max(n_vec * xs, 4), np.uint8)
        for t in range(n_vec):
            xbuf[t * xs:t * xs + cols * 4] = x[t].view(np.uint8)
        xb = self.be.import_host_readonly(xbuf)
        ys = y_stride or rows * 4
        sentinel = np.float32(-12345.625)
        ybytes = max(n_vec * ys, 4) + 2 * y_guard * 4
        yb = self.be.allocate(ybytes)
        fill = np.full(ybytes // 4, sentinel, np.float32)
        self.be.upload(self.st, hb.TensorRef.of(yb), fill)
        a = hb.GemvArgs(wtype, hb.TensorRef(wb, w_offset, 0, w_stride), hb.TensorRef(xb, 0, 0, x_stride),
                        hb.TensorRef(yb, y_guard * 4, 0, y_stride), rows, cols, n_vec, variant, allow_gemm=allow_gemm)
        self.be.gemv(self.st, a)
        out = np.empty(ybytes // 4, np.float32)
        self.be.download(self.st, hb.TensorRef.of(yb), out)
        self.st.wait()
        body = out[y_guard:len(out) - y_guard] if y_guard else out
        y = np.empty((n_vec, rows), np.float32)
        for t in range(n_vec):
            y[t] = body[t * ys // 4:t * ys // 4 + rows]
        if y_guard:
            assert np.all(out[:y_guard] == sentinel) and np.all(out[len(out) - y_guard:] == sentinel), "y guard band overwritten"
            for t in range(n_vec):  # the gaps between strided rows must survive too
                gap = body[t * ys // 4 + rows:(t + 1) * ys // 4]
                assert np.all(gap == sentinel), "y row padding overwritten"
        return y

    def dequant(self, wtype, w, n_rows, cols, ids=None):
        wb = self.be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
        n_ids = n_rows if ids is None else len(ids)
        ob = self.be.allocate(max(n_ids * cols * 4, 4))
        ib = self.be.import_host_readonly(np.asarray(ids, np.int32)) if ids is not None else None
        sb = self.be.allocate(4)
        a = hb.GetRowsArgs(wtype, hb.TensorRef.of(wb), hb.TensorRef.of(ib) if ib else hb.TensorRef(), hb.TensorRef.of(ob),
                           n_rows, cols, n_ids)
        self.be.get_rows(self.st, a, status=sb)
        out = np.empty((n_ids, cols), np.float32)
        status = np.zeros(1, np.uint32)
        self.be.download(self.st, hb.TensorRef.of(ob), out)
        self.be.download(self.st, hb.TensorRef.of(sb), status)
        self.st.wait()
        return out, int(status[0])

    def lm_head(self, wtype, w, x, rows, cols, *, variant=0, valid_rows=0, want_logits=True, want_ids=True, row_offset=0):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
        n_vec = x.shape[0]
        wb = self.be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
        xb = self.be.import_host_readonly(x)
        lb = self.be.allocate(n_vec * rows * 4) if want_logits else None
        rb = self.be.allocate(n_vec * 12)
        ib = self.be.allocate(n_vec * 4) if want_ids else None
        g = hb.GemvArgs(wtype, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(lb) if lb else hb.TensorRef(), rows, cols,
                        n_vec, variant)
        a = hb.LmHeadArgs(g, hb.TensorRef.of(rb), valid_rows, hb.TensorRef.of(ib) if ib else hb.TensorRef(), row_offset)
        self.be.lm_head(self.st, a)
        res = np.zeros((n_vec, 3), np.uint32)
        self.be.download(self.st, hb.TensorRef.of(rb), res)
        logits = np.zeros((n_vec, rows), np.float32) if want_logits else None
        ids = np.zeros(n_vec, np.int32) if want_ids else None
        if want_logits:
            self.be.download(self.st, hb.TensorRef.of(lb), logits)
        if want_ids:
            self.be.download(self.st, hb.TensorRef.of(ib), ids)
        self.st.wait()
        return res, logits, ids


def summation_bound(checker_dequant, wtype, w, x, rows, cols, depth):
    """(d_cpu + d_gpu) * u * sum|x_i w_i| per output: the reference's derived bound for reordered fp32 sums
    (tests/unit/hip/test_hip_gemv.cpp:9-15), with d = number of roundings on the longest path."""
    wf = checker_dequant(wtype, w, rows * cols).reshape(rows, cols).astype(np.float64)
    s = np.abs(np.asarray(x, np.float64)) @ np.abs(wf).T
    return depth * 2.0**-24 * s


def half_steps(x: np.ndarray) -> np.ndarray:
    """Half a quantisation step of every element of x (rows of a multiple of 256 floats) in the int8 tensor-core family: the kernels
    scale a super-block by the power of two s that puts its largest magnitude m in (2^14, 32639] and round x * s to an integer."""
    x = np.asarray(x, np.float64)
    blocks = np.abs(x).reshape(x.shape[0], -1, 256)
    m = blocks.max(axis=2)
    with np.errstate(divide="ignore"):
        se = np.where(m > 0, 14 - np.floor(np.log2(np.where(m > 0, m, 1.0))), 0.0)
    se = np.clip(se, -100, 100)
    se = np.where(m * np.exp2(se) > 32639.0, se - 1, se)
    return np.repeat(0.5 * np.exp2(-se), 256, axis=1)


def rounded_operand_bound(checker, t, w, x, n, k):
    """sum |w_i| * (half a quantisation step of x_i) plus the reordered-summation bound: what a kernel that rounds x to 16-bit fixed
    point and then sums in its own order may differ from the CPU backend by."""
    wf = checker.dequantize(t, w, n * k).reshape(n, k).astype(np.float64)
    return half_steps(x) @ np.abs(wf).T + summation_bound(checker.dequantize, t, w, x, n, k, depth=2 * (k // 8 + 8))
