"""ctypes/numpy front end of the CPU oracle (``libdsuf_oracle.so``, built by ``oracle/Makefile``).

TEST INFRASTRUCTURE ONLY.  Importers: ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline /
reference legs of ``bench.py``.  The product package never imports this module.

bf16 tensors travel as ``uint16`` numpy arrays, e4m3/e2m1/UE8M0 as ``uint8``.
"""
import ctypes as C
import os
import subprocess

import numpy as np

MODE_MX, MODE_DS = 0, 1
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    subprocess.run(["make", "-C", _HERE, "--no-print-directory"], check=True, capture_output=True)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libdsuf_oracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.dsufo_e4m3_to_f32.restype = C.c_float
        L.dsufo_e4m3_to_f32.argtypes = [C.c_uint8]
        L.dsufo_e8m0_to_f32.restype = C.c_float
        L.dsufo_e8m0_to_f32.argtypes = [C.c_uint8]
        L.dsufo_e2m1_to_f32.restype = C.c_float
        L.dsufo_e2m1_to_f32.argtypes = [C.c_uint8]
        for f in (L.dsufo_f32_to_e4m3, L.dsufo_f32_to_e4m3_fast, L.dsufo_f32_to_e2m1):
            f.restype = C.c_uint8
            f.argtypes = [C.c_float]
        L.dsufo_round_scale_pow2.restype = C.c_float
        L.dsufo_round_scale_pow2.argtypes = [C.c_float, C.c_float]
        L.dsufo_f32_to_bf16.restype = C.c_uint16
        L.dsufo_f32_to_bf16.argtypes = [C.c_float]
        L.dsufo_permute_plan.restype = C.c_int
        L.dsufo_num_threads.restype = C.c_int
        L.dsufo_set_num_threads.restype = C.c_int
        L.dsufo_set_num_threads.argtypes = [C.c_int]
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


def f32_to_bf16(a):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_to_f32(a):
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_lut():
    return np.array([lib().dsufo_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)


def e2m1_lut():
    return np.array([lib().dsufo_e2m1_to_f32(i) for i in range(16)], dtype=np.float32)


def act_quant(mode, x_bf16):
    x = _c(x_bf16, np.uint16)
    m, k = x.shape
    blk = 32 if mode == MODE_MX else 128
    q = np.empty((m, k), np.uint8)
    s = np.empty((m, k // blk), np.uint8 if mode == MODE_MX else np.float32)
    lib().dsufo_act_quant(C.c_int(mode), _p(x), C.c_int(k), C.c_int(m), C.c_int(k), _p(q), _p(s))
    return q, s


def row_sumsq(x_bf16):
    """tc_row_sumsq (crates/kernels/cu/tcgemm.cu:341-355), summation order restated exactly."""
    x = _c(x_bf16, np.uint16)
    m, k = x.shape
    out = np.empty(m, np.float32)
    lib().dsufo_row_sumsq(_p(x), C.c_int(k), C.c_int(m), C.c_int(k), _p(out))
    return out


def act_quant_prenorm(mode, x_bf16, norm_w_bf16, sumsq, eps):
    """tc_quant_rows with RMS pre-normalisation (crates/kernels/cu/tcgemm.cu:300-340)."""
    x = _c(x_bf16, np.uint16)
    w = _c(norm_w_bf16, np.uint16)
    ss = _c(sumsq, np.float32)
    m, k = x.shape
    blk = 32 if mode == MODE_MX else 128
    q = np.empty((m, k), np.uint8)
    s = np.empty((m, k // blk), np.uint8 if mode == MODE_MX else np.float32)
    lib().dsufo_act_quant_prenorm(C.c_int(mode), _p(x), C.c_int(k), C.c_int(m), C.c_int(k), _p(w), _p(ss), C.c_float(eps), _p(q), _p(s))
    return q, s


def quant_fp8_weight(mode, w_bf16):
    w = _c(w_bf16, np.uint16)
    n, k = w.shape
    blk = 32 if mode == MODE_MX else 128
    q = np.empty((n, k), np.uint8)
    s = np.empty((n // blk, k // blk), np.uint8 if mode == MODE_MX else np.float32)
    lib().dsufo_quant_fp8_weight(C.c_int(mode), _p(w), C.c_int(n), C.c_int(k), _p(q), _p(s))
    return q, s


def quant_fp4_weight(w_bf16):
    w = _c(w_bf16, np.uint16)
    n, k = w.shape
    codes = np.empty((n, k // 2), np.uint8)
    s = np.empty((n, k // 32), np.uint8)
    lib().dsufo_quant_fp4_weight(_p(w), C.c_int(n), C.c_int(k), _p(codes), _p(s))
    return codes, s


def gemm_fp8(mode, wq, ws, xq, xs, alpha=1.0):
    """Returns (out_bf16 [m][n] as uint16, out_f32 [m][n])."""
    wq, xq = _c(wq, np.uint8), _c(xq, np.uint8)
    sdt = np.uint8 if mode == MODE_MX else np.float32
    ws, xs = _c(ws, sdt), _c(xs, sdt)
    n, k = wq.shape
    m = xq.shape[0]
    ob = np.empty((m, n), np.uint16)
    of = np.empty((m, n), np.float32)
    lib().dsufo_gemm_fp8(C.c_int(mode), _p(wq), _p(ws), C.c_int(n), C.c_int(k), _p(xq), _p(xs), C.c_int(m),
                         C.c_float(alpha), _p(ob), _p(of), C.c_int(n))
    return ob, of


def gemm_fp4(act_mode, codes, wscale, xq, xs):
    codes, wscale, xq = _c(codes, np.uint8), _c(wscale, np.uint8), _c(xq, np.uint8)
    xs = _c(xs, np.uint8 if act_mode == MODE_MX else np.float32)
    n, k = codes.shape[0], codes.shape[1] * 2
    m = xq.shape[0]
    of = np.empty((m, n), np.float32)
    lib().dsufo_gemm_fp4(C.c_int(act_mode), _p(codes), _p(wscale), C.c_int(n), C.c_int(k), _p(xq), _p(xs), C.c_int(m),
                         _p(of), C.c_int(n))
    return of


def route(score_fn, scores, bias, topk, route_scale=1.0):
    scores = _c(scores, np.float32)
    t, e = scores.shape
    bias = None if bias is None else _c(bias, np.float32)
    ids = np.empty((t, topk), np.int32)
    w = np.empty((t, topk), np.float32)
    lib().dsufo_route(C.c_int(score_fn), _p(scores), _p(bias), C.c_int(t), C.c_int(e), C.c_int(topk),
                      C.c_float(route_scale), _p(ids), _p(w))
    return ids, w


def permute_plan(ids, n_exp, tile_rows=128):
    ids = _c(ids, np.int32).reshape(-1)
    p = ids.size
    off = np.empty(n_exp + 1, np.int32)
    row_pair = np.empty(p, np.int32)
    pair_row = np.empty(p, np.int32)
    tiles = np.zeros((p // tile_rows + n_exp + 1, 4), np.int32)
    nt = lib().dsufo_permute_plan(_p(ids), C.c_int(p), C.c_int(n_exp), C.c_int(tile_rows), _p(off), _p(row_pair),
                                  _p(pair_row), _p(tiles))
    return off, row_pair, pair_row, tiles[:nt].copy()


def moe_layer(act_mode, x_bf16, ids, w, w13c, w13s, w2c, w2s, swiglu_limit=0.0, shared=None, e_lo=0, e_hi=None,
              want_act=False, want_ypair=False):
    """w13c [E][2I][H/2], w13s [E][2I][H/32], w2c [E][H][I/2], w2s [E][H][I/32]. Returns dict."""
    x = _c(x_bf16, np.uint16)
    t, h = x.shape
    ids, w = _c(ids, np.int32), _c(w, np.float32)
    topk = ids.shape[1]
    w13c, w13s, w2c, w2s = (_c(a, np.uint8) for a in (w13c, w13s, w2c, w2s))
    n_exp, two_i = w13c.shape[0], w13c.shape[1]
    inter = two_i // 2
    e_hi = n_exp if e_hi is None else e_hi
    yb = np.empty((t, h), np.uint16)
    yf = np.empty((t, h), np.float32)
    act = np.empty((t * topk, inter), np.uint16) if want_act else None
    yp = np.empty((t * topk, h), np.float32) if want_ypair else None
    sh = None if shared is None else _c(shared, np.uint16)
    lib().dsufo_moe_layer(C.c_int(act_mode), _p(x), C.c_int(t), C.c_int(h), C.c_int(inter), C.c_int(topk), _p(ids), _p(w),
                          _p(w13c), _p(w13s), _p(w2c), _p(w2s), C.c_float(swiglu_limit), _p(sh), C.c_int(e_lo),
                          C.c_int(e_hi), _p(yb), _p(yf), _p(act), _p(yp))
    return {"y_bf16": yb, "y_f32": yf, "act_bf16": act, "ypair": yp}


def matmul_f32(w_deq, x_deq):
    w_deq, x_deq = _c(w_deq, np.float32), _c(x_deq, np.float32)
    n, k = w_deq.shape
    m = x_deq.shape[0]
    out = np.empty((m, n), np.float32)
    lib().dsufo_matmul_f32(_p(w_deq), _p(x_deq), C.c_int(n), C.c_int(k), C.c_int(m), _p(out))
    return out


def dequant_fp8(mode, q, s):
    """fp32 dequantization of an FP8 matrix with its block scales (row blocks only for activations)."""
    lut = e4m3_lut()
    v = lut[np.asarray(q)]
    blk = 32 if mode == MODE_MX else 128
    s = np.asarray(s)
    sf = (s.astype(np.uint32) << 23).view(np.float32) if mode == MODE_MX else s.astype(np.float32)
    if sf.shape[0] == v.shape[0]:  # per-row scales (activations)
        return v * np.repeat(sf, blk, axis=1)
    return v * np.repeat(np.repeat(sf, blk, axis=0), blk, axis=1)


def dequant_fp4(codes, s):
    lut = e2m1_lut()
    codes = np.asarray(codes)
    n, kh = codes.shape
    v = np.empty((n, kh * 2), np.float32)
    v[:, 0::2] = lut[codes & 15]
    v[:, 1::2] = lut[codes >> 4]
    sf = (np.asarray(s).astype(np.uint32) << 23).view(np.float32)
    return v * np.repeat(sf, 32, axis=1)


def rope_rows(v_f32, cos, sin, pos0, head, off, n_first=None):
    """The fused rotary embedding of the reference's GEMV epilogue (crates/kernels/cu/gemv.cu:508-516) applied to fp32
    results v [m][n]: columns r < n_first (default: all) with (r % head) >= off are rotated in (even, odd) pairs:
    a = bf16(v[r]), b = bf16(v[r+1]); out[r] = fma(a, c, -(b*s)), out[r+1] = fma(a, s, b*c) with c / s =
    cos / sin[pos0 + token][((r % head) - off) / 2]; fp32 in, bf16-rounded fp32 out (every column rounded to bf16)."""
    v = np.asarray(v_f32, np.float32)
    m, n = v.shape
    n_first = n if n_first is None else n_first
    out = bf16_to_f32(f32_to_bf16(v)).astype(np.float32)
    r = np.arange(0, n_first, 2)
    sel = r[(r % head) >= off]
    f = ((sel % head) - off) // 2
    for t in range(m):
        a, b = out[t, sel].astype(np.float64), out[t, sel + 1].astype(np.float64)
        c, s_ = cos[pos0 + t, f].astype(np.float64), sin[pos0 + t, f].astype(np.float64)
        bs, bc = (b * s_).astype(np.float32).astype(np.float64), (b * c).astype(np.float32).astype(np.float64)
        o0, o1 = (a * c - bs).astype(np.float32), (a * s_ + bc).astype(np.float32)
        out[t, sel] = bf16_to_f32(f32_to_bf16(o0))
        out[t, sel + 1] = bf16_to_f32(f32_to_bf16(o1))
    return out


def lm_head(w_bf16, x_bf16, alpha=1.0):
    """Output-head logits fp32 [m][n] = alpha * x . w^T over bf16 operands with fp32 accumulation
    (gemv_bf16_persist_body, crates/kernels/cu/gemv.cu:542-650; the accumulation order inside a row is the kernel's own,
    so comparisons carry a tolerance)."""
    return (matmul_f32(bf16_to_f32(w_bf16), bf16_to_f32(x_bf16)) * np.float32(alpha)).astype(np.float32)


def sampling_records(logits, temperature, valid_rows=0, id_offset=0):
    """Per (token, quad of 64 vocabulary rows) the 20-float record of crates/kernels/cu/gemv.cu:651-688:
    [0] max z, [1] sum exp(z - max), [2] 9th largest z, [3..10] the 8 largest z (descending), [11..18] their ids as int
    bits (equal values: lower id first), [19] 0; z = logit * (1 / temperature) in fp32 for rows < valid_rows (0: all),
    -inf above; id = row + id_offset.  Plain loops over quads: small inputs only."""
    logits = np.asarray(logits, np.float32)
    m, n = logits.shape
    assert n % 64 == 0
    vloc = valid_rows if valid_rows > 0 else n
    inv_t = np.float32(1.0) / np.float32(temperature)
    rec = np.zeros((m, n // 64, 20), np.float32)
    ids_view = rec.view(np.int32)
    for t in range(m):
        for q in range(n // 64):
            rows = np.arange(q * 64, q * 64 + 64)
            z = np.where(rows < vloc, logits[t, rows] * inv_t, np.float32(-np.inf)).astype(np.float32)
            order = np.lexsort((rows, -z.astype(np.float64)))     # by z descending, then by id ascending
            top = order[:9]
            zmax = z[top[0]]
            rec[t, q, 0] = zmax
            with np.errstate(invalid="ignore"):
                e = np.where(np.isneginf(z), np.float32(0), np.exp((z - zmax).astype(np.float32), dtype=np.float32))
            rec[t, q, 1] = np.float32(e.astype(np.float64).sum())
            rec[t, q, 2] = z[top[8]]
            rec[t, q, 3:11] = z[top[:8]]
            ids_view[t, q, 11:19] = rows[top[:8]] + id_offset
    return rec


def num_threads():
    return lib().dsufo_num_threads()


def use_all_host_cores():
    """Sets the OpenMP thread count to the cores this process may run on (a launcher may have exported
    OMP_NUM_THREADS=1); returns the count in force."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    return lib().dsufo_set_num_threads(n)
