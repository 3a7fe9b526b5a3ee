"""Host-side mirror of deepseek-ultrafast's kernel call surface over libdsuf_qmm (C ABI, include/dsuf_qmm.h).

The reference's host side is Rust (crates/engine/src/ops.rs); no Rust toolchain exists in this build
environment, so the same operator surface is mirrored here in Python over ctypes.  Names follow the reference:
``gemv`` (ops.rs:331), ``moe_route_tokens`` / ``moe_perm`` / ``moe_gather_quant`` (cu/ops.cu:615, cu/tcmoe.cu:19,88),
``moe_gemv`` (ops.rs:482), ``ffn`` (crates/engine/src/model.rs:3497).  PyTorch is used only to own device memory
and streams; every computation happens in the library's CUDA kernels.  There is no fallback: if the shared
library is missing or the device is not sm_100, construction fails.
"""
import ctypes as C
import os

import numpy as np

MODE_MX, MODE_DS = 0, 1
FMT_FP8, FMT_FP4 = 0, 1
SCORE_IDENTITY, SCORE_SOFTMAX, SCORE_SQRT_SOFTPLUS = 0, 1, 2
EPI_STORE, EPI_SWIGLU, EPI_SQRT_SOFTPLUS, EPI_ACCUMULATE = 0, 1, 2, 3   # dsuf_gemm_opts.epilogue

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdsuf_qmm.so")
_LIB = None


class DsufError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"dsuf error {code}: {msg}")
        self.code = code


class WeightDesc(C.Structure):
    _fields_ = [("fmt", C.c_int32), ("mode", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("n_experts", C.c_int32),
                ("gate_up", C.c_int32), ("tiles", C.c_uint64), ("scales_ds", C.c_uint64)]


class PlanStruct(C.Structure):
    _fields_ = [("expert_off", C.c_uint64), ("row_pair", C.c_uint64), ("pair_row", C.c_uint64), ("row_w", C.c_uint64),
                ("tiles", C.c_uint64), ("ntiles", C.c_uint64), ("scratch", C.c_uint64), ("p", C.c_int32),
                ("n_exp", C.c_int32), ("tile_rows", C.c_int32), ("max_tiles", C.c_int32)]


class GemmOpts(C.Structure):
    _fields_ = [("alpha", C.c_float), ("out_f32", C.c_int32), ("n_split", C.c_int32), ("ldo2", C.c_int32), ("out2", C.c_uint64),
                ("epilogue", C.c_int32), ("swiglu_limit", C.c_float), ("rope_cos", C.c_uint64), ("rope_sin", C.c_uint64),
                ("rope_pos", C.c_uint64), ("rope_head", C.c_int32), ("rope_off", C.c_int32)]


class SamplingOpts(C.Structure):
    _fields_ = [("records", C.c_uint64), ("temperature", C.c_float), ("valid_rows", C.c_int32), ("id_offset", C.c_int32)]


class TensorInfo(C.Structure):
    _fields_ = [("dtype", C.c_char * 16), ("rank", C.c_int32), ("shape", C.c_int64 * 8), ("data", C.c_void_p), ("nbytes", C.c_size_t)]


class DevStatus(C.Structure):
    _fields_ = [("code", C.c_int32), ("kernel", C.c_int32), ("cta", C.c_int32), ("where", C.c_int32)]


# name -> (restype, argtypes); also the list the symbol-export test walks
ABI = {
    "dsuf_ctx_create": (C.c_int32, [C.c_int32, C.POINTER(C.c_void_p)]),
    "dsuf_ctx_destroy": (C.c_int32, [C.c_void_p]),
    "dsuf_last_error": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "dsuf_ctx_set_pdl": (C.c_int32, [C.c_void_p, C.c_int32]),
    "dsuf_ctx_set_decode_path": (C.c_int32, [C.c_void_p, C.c_int32]),
    "dsuf_status_poll": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(DevStatus)]),
    "dsuf_sm_count": (C.c_int32, [C.c_void_p]),
    "dsuf_ctx_set_wait_budget_us": (C.c_int32, [C.c_void_p, C.c_int64]),
    "dsuf_ctx_set_prenorm_rsqrt": (C.c_int32, [C.c_void_p, C.c_int32]),
    "dsuf_ctx_set_dense_ksplit": (C.c_int32, [C.c_void_p, C.c_int32]),
    "dsuf_ctx_set_stage_pairs": (C.c_int32, [C.c_void_p, C.c_int32]),
    "dsuf_quant_fp8_weight_host": (C.c_int32, [C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "dsuf_quant_fp4_weight_host": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "dsuf_packed_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "dsuf_pack_fp8_weight": (C.c_int32, [C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "dsuf_pack_fp8_weight_gate_up": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "dsuf_pack_fp4_weight": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "dsuf_ckpt_open": (C.c_int32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "dsuf_ckpt_close": (C.c_int32, [C.c_void_p]),
    "dsuf_ckpt_last_error": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "dsuf_ckpt_count": (C.c_int64, [C.c_void_p]),
    "dsuf_ckpt_tensor": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(TensorInfo)]),
    "dsuf_ckpt_load_fp8_dense": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "dsuf_ckpt_load_fp4_experts": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "dsuf_weight_create": (C.c_int32, [C.c_void_p, C.POINTER(WeightDesc), C.POINTER(C.c_void_p)]),
    "dsuf_weight_destroy": (C.c_int32, [C.c_void_p]),
    "dsuf_row_sumsq": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int32, C.c_int32, C.c_int32, C.c_uint64]),
    "dsuf_act_quant_fp8_prenorm": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint64, C.c_int32, C.c_int32, C.c_int32,
                                               C.c_uint64, C.c_uint64, C.c_float, C.c_uint64, C.c_uint64]),
    "dsuf_ep_flag_bytes": (C.c_size_t, [C.c_int32]),
    "dsuf_ep_allreduce_bf16": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.c_int32, C.c_int32,
                                           C.c_int64, C.c_uint64, C.c_uint64]),
    "dsuf_ep_allgather_cols_bf16": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.c_int32, C.c_int32,
                                                C.c_int32, C.c_int32, C.c_uint64, C.c_uint64]),
    "dsuf_ep_combine_bf16": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int32, C.c_int32, C.c_int32,
                                         C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.c_int32, C.c_int32, C.c_uint64, C.c_uint64]),
    "dsuf_ep_combine_quant_bf16": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int32, C.c_int32, C.c_int32,
                                               C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.c_int32, C.c_int32, C.c_uint64, C.c_uint64,
                                               C.c_int32, C.c_uint64, C.c_uint64]),
    "dsuf_act_quant_fp8": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint64, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_uint64, C.c_uint64]),
    "dsuf_gemm_workspace_bytes": (C.c_size_t, [C.c_void_p]),
    "dsuf_workspace_init": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_size_t]),
    "dsuf_gemm_fp8": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int32, C.c_uint64,
                                  C.c_int32, C.c_float, C.c_uint64]),
    "dsuf_gemm_fp8_ex": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int32, C.c_uint64,
                                     C.c_int32, C.POINTER(GemmOpts), C.c_uint64]),
    "dsuf_gemm_fp8_static": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int32, C.c_uint64,
                                         C.c_int32, C.c_float]),
    "dsuf_lm_head_bf16": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int32, C.c_int32, C.c_uint64, C.c_int32, C.c_int32, C.c_float,
                                      C.c_uint64, C.c_int32, C.POINTER(SamplingOpts)]),
    "dsuf_probe_tensor_rate": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_double)]),
    "dsuf_moe_route": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint64, C.c_uint64, C.c_int32, C.c_int32,
                                   C.c_int32, C.c_float, C.c_uint64, C.c_uint64]),
    "dsuf_moe_plan_scratch_ints": (C.c_size_t, [C.c_int32, C.c_int32]),
    "dsuf_moe_permute_plan": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int32, C.POINTER(PlanStruct)]),
    "dsuf_moe_route_plan_gather": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint64, C.c_uint64, C.c_int32, C.c_int32, C.c_int32,
                                               C.c_float, C.c_uint64, C.c_uint64, C.c_int32, C.POINTER(PlanStruct), C.c_int32, C.c_uint64,
                                               C.c_int32, C.c_int32, C.c_uint64, C.c_uint64]),
    "dsuf_moe_gather_quant_prenorm": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint64, C.c_int32, C.c_int32, C.c_int32,
                                                  C.c_int32, C.c_void_p, C.c_uint64, C.c_uint64, C.c_float, C.c_uint64, C.c_uint64]),
    "dsuf_moe_gather_quant": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint64, C.c_int32, C.c_int32, C.c_int32,
                                          C.c_int32, C.POINTER(PlanStruct), C.c_uint64, C.c_uint64]),
    "dsuf_moe_w13_swiglu": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(PlanStruct), C.c_uint64,
                                        C.c_uint64, C.c_float, C.c_uint64]),
    "dsuf_moe_w2": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(PlanStruct), C.c_uint64,
                                C.c_uint64, C.c_uint64]),
    "dsuf_moe_unpermute": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(PlanStruct), C.c_uint64, C.c_uint64, C.c_int32,
                                       C.c_int32, C.c_int32, C.c_uint64, C.c_int32]),
    "dsuf_moe_unpermute_quant": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(PlanStruct), C.c_uint64, C.c_uint64, C.c_int32, C.c_int32,
                                             C.c_int32, C.c_uint64, C.c_int32, C.c_int32, C.c_uint64, C.c_uint64]),
}


def lib():
    """Loads libdsuf_qmm.so; raises if it has not been built (there is deliberately no other code path)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise DsufError(-2, f"{LIB_PATH} is missing: build it with `python deepseek-ultrafast_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in ABI.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _LIB = L
    return _LIB


def _np_ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ------------------------------------------------------------------ host formats (no GPU)
def quant_fp8_weight_host(mode, w_bf16):
    w = np.ascontiguousarray(w_bf16, dtype=np.uint16)
    n, k = w.shape
    blk = 32 if mode == MODE_MX else 128
    codes = np.empty((n, k), np.uint8)
    scales = np.empty((n // blk, k // blk), np.uint8 if mode == MODE_MX else np.float32)
    rc = lib().dsuf_quant_fp8_weight_host(mode, _np_ptr(w), n, k, _np_ptr(codes), _np_ptr(scales))
    if rc:
        raise DsufError(rc, "dsuf_quant_fp8_weight_host")
    return codes, scales


def quant_fp4_weight_host(w_bf16):
    w = np.ascontiguousarray(w_bf16, dtype=np.uint16)
    n, k = w.shape
    codes = np.empty((n, k // 2), np.uint8)
    scales = np.empty((n, k // 32), np.uint8)
    rc = lib().dsuf_quant_fp4_weight_host(_np_ptr(w), n, k, _np_ptr(codes), _np_ptr(scales))
    if rc:
        raise DsufError(rc, "dsuf_quant_fp4_weight_host")
    return codes, scales


def pack_fp8_weight(mode, codes, scales):
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    n, k = codes.shape
    out = np.empty(lib().dsuf_packed_bytes(FMT_FP8, mode, n, k), np.uint8)
    sc = None if scales is None else np.ascontiguousarray(scales)
    rc = lib().dsuf_pack_fp8_weight(mode, _np_ptr(codes), _np_ptr(sc), n, k, _np_ptr(out))
    if rc:
        raise DsufError(rc, "dsuf_pack_fp8_weight")
    return out


def pack_fp4_weight(codes, scales, gate_up):
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    n, k = codes.shape[0], codes.shape[1] * 2
    out = np.empty(lib().dsuf_packed_bytes(FMT_FP4, MODE_MX, n, k), np.uint8)
    rc = lib().dsuf_pack_fp4_weight(_np_ptr(codes), _np_ptr(scales), n, k, int(bool(gate_up)), _np_ptr(out))
    if rc:
        raise DsufError(rc, "dsuf_pack_fp4_weight")
    return out


class Checkpoint:
    """Checkpoint (crates/model/src/st.rs:17-106) + the weight loaders (crates/engine/src/weights.rs:254-276, 421-446):
    a directory of .safetensors files (or one file), read-only mapped; tensors by name, FP8 dense weights and FP4 experts
    as this library's tile records."""

    def __init__(self, path):
        h = C.c_void_p()
        rc = lib().dsuf_ckpt_open(os.fsencode(path), C.byref(h))
        self.h = h
        if rc:
            msg = self._err()
            self.close()
            raise DsufError(rc, msg)

    def _err(self):
        buf = C.create_string_buffer(512)
        lib().dsuf_ckpt_last_error(self.h, buf, 512)
        return buf.value.decode()

    def _check(self, rc):
        if rc:
            raise DsufError(rc, self._err())

    def close(self):
        if self.h:
            lib().dsuf_ckpt_close(self.h)
            self.h = None

    def __len__(self):
        return int(lib().dsuf_ckpt_count(self.h))

    def tensor(self, name):
        """(dtype string, shape tuple, uint8 numpy view of the bytes inside the mapping)."""
        ti = TensorInfo()
        self._check(lib().dsuf_ckpt_tensor(self.h, name.encode(), C.byref(ti)))
        raw = np.ctypeslib.as_array(C.cast(ti.data, C.POINTER(C.c_uint8)), shape=(ti.nbytes,)) if ti.nbytes else np.empty(0, np.uint8)
        return ti.dtype.decode(), tuple(ti.shape[i] for i in range(ti.rank)), raw

    def fp8_dense_tiles(self, name, rows=None):
        """Loader::fp8: MX tile records (host numpy) of `{name}.weight` / `{name}.scale`, optionally rows [r0, r1)."""
        _, shape, _ = self.tensor(name + ".weight")
        n, k = shape
        r0, r1 = rows if rows is not None else (0, n)
        out = np.empty(lib().dsuf_packed_bytes(FMT_FP8, MODE_MX, r1 - r0, k), np.uint8)
        self._check(lib().dsuf_ckpt_load_fp8_dense(self.h, name.encode(), n, k, r0, r1, _np_ptr(out)))
        return out, r1 - r0, k

    def fp4_expert_tiles(self, prefix, e0, e1, dim, inter):
        """Experts e0 .. e1-1 of `{prefix}.ffn.experts.{e}`: (w13 records, w2 records) as host numpy arrays."""
        per13 = lib().dsuf_packed_bytes(FMT_FP4, MODE_MX, 2 * inter, dim)
        per2 = lib().dsuf_packed_bytes(FMT_FP4, MODE_MX, dim, inter)
        o13, o2 = np.empty((e1 - e0) * per13, np.uint8), np.empty((e1 - e0) * per2, np.uint8)
        self._check(lib().dsuf_ckpt_load_fp4_experts(self.h, prefix.encode(), e0, e1, dim, inter, _np_ptr(o13), _np_ptr(o2)))
        return o13, o2

    def load_fp8_dense(self, ctx, name, rows=None):
        """`{name}` as a device Weight (MX geometry, the checkpoint's own)."""
        tiles, n, k = self.fp8_dense_tiles(name, rows)
        return Weight(ctx, FMT_FP8, MODE_MX, n, k, 1, False, ctx.torch.from_numpy(tiles).to(ctx.device))

    def load_experts(self, ctx, prefix, e0, e1, dim, inter):
        """(W13, W2) device Weights of the experts e0 .. e1-1 (an expert-parallel rank passes its own range)."""
        o13, o2 = self.fp4_expert_tiles(prefix, e0, e1, dim, inter)
        t = ctx.torch
        return (Weight.experts_fp4_packed(ctx, t.from_numpy(o13).to(ctx.device), 2 * inter, dim, e1 - e0, True),
                Weight.experts_fp4_packed(ctx, t.from_numpy(o2).to(ctx.device), dim, inter, e1 - e0, False))


# ------------------------------------------------------------------ device side
class Ctx:
    """dsuf_ctx wrapper: one per device (Device::new + ops::hw(), crates/cuda/src/lib.rs:52, ops.rs:205)."""

    def __init__(self, device=0, pdl=False, tcgen05=True):
        import torch
        self.torch = torch
        self.device = torch.device("cuda", device)
        h = C.c_void_p()
        rc = lib().dsuf_ctx_create(device, C.byref(h))
        if rc:
            raise DsufError(rc, "dsuf_ctx_create failed (needs an sm_100 GPU)")
        self.h = h
        if pdl:
            self.check(lib().dsuf_ctx_set_pdl(self.h, 1))
        self.set_decode_path(tcgen05)
        nbytes = lib().dsuf_gemm_workspace_bytes(self.h)
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.check(lib().dsuf_workspace_init(self.h, self.stream(), self.workspace.data_ptr(), nbytes))
        self.sm_count = lib().dsuf_sm_count(self.h)

    def set_decode_path(self, tcgen05):
        """True: tcgen05 streaming kernels for decode shapes; False: the mma.sync streaming kernels."""
        self.check(lib().dsuf_ctx_set_decode_path(self.h, 1 if tcgen05 else 0))
        self.tcgen05 = bool(tcgen05)

    def set_stage_pairs(self, enabled):
        """Two tile records per ring stage in the decode expert GEMMs (default on)."""
        self.check(lib().dsuf_ctx_set_stage_pairs(self.h, 1 if enabled else 0))

    def set_dense_ksplit(self, enabled):
        """Cluster K-split for dense decode GEMVs with few row tiles (default on)."""
        self.check(lib().dsuf_ctx_set_dense_ksplit(self.h, 1 if enabled else 0))

    def set_prenorm_rsqrt_approx(self, approximate):
        """True: the pre-normalising quantizers use the GPU's approximate rsqrt, as the reference's kernels do."""
        self.check(lib().dsuf_ctx_set_prenorm_rsqrt(self.h, 1 if approximate else 0))

    def set_wait_budget_us(self, microseconds):
        """Upper bound of the peer-exchange kernels' wait for a peer (they report a time-out in the status word after it)."""
        self.check(lib().dsuf_ctx_set_wait_budget_us(self.h, int(microseconds)))

    def stream(self):
        return C.c_void_p(self.torch.cuda.current_stream(self.device).cuda_stream)

    def check(self, rc):
        if rc:
            buf = C.create_string_buffer(512)
            lib().dsuf_last_error(self.h, buf, 512)
            raise DsufError(rc, buf.value.decode())

    def status(self):
        st = DevStatus()
        self.check(lib().dsuf_status_poll(self.h, self.stream(), C.byref(st)))
        return st

    def close(self):
        if self.h:
            lib().dsuf_ctx_destroy(self.h)
            self.h = None


class Weight:
    """Weight{fmt,w,s,n,k} / Experts (ops.rs:6-39, crates/engine/src/weights.rs:82-92) over a packed tile image."""

    def __init__(self, ctx, fmt, mode, n, k, n_experts, gate_up, tiles, scales_ds=None):
        self.ctx, self.fmt, self.mode, self.n, self.k = ctx, fmt, mode, n, k
        self.n_experts, self.gate_up = n_experts, gate_up
        self.tiles, self.scales_ds = tiles, scales_ds  # keep the device tensors alive
        d = WeightDesc(fmt, mode, n, k, n_experts, int(bool(gate_up)), tiles.data_ptr(),
                       scales_ds.data_ptr() if scales_ds is not None else 0)
        h = C.c_void_p()
        ctx.check(lib().dsuf_weight_create(ctx.h, C.byref(d), C.byref(h)))
        self.h = h

    @staticmethod
    def dense_fp8(ctx, mode, codes, scales):
        """codes u8 [n][k]; scales MX u8 [n/32][k/32] or DS f32 [n/128][k/128] (host arrays)."""
        t = ctx.torch
        n, k = codes.shape
        tiles = t.from_numpy(pack_fp8_weight(mode, codes, scales if mode == MODE_MX else None)).to(ctx.device)
        sds = t.from_numpy(np.ascontiguousarray(scales, np.float32)).to(ctx.device) if mode == MODE_DS else None
        return Weight(ctx, FMT_FP8, mode, n, k, 1, False, tiles, sds)

    @staticmethod
    def dense_fp8_gate_up(ctx, codes, scales):
        """The FP8 shared expert's gate/up weight: MX codes u8 [2*inter][k] (gate rows, then up rows) + u8 [2*inter/32][k/32]
        scales, rows interleaved for the SwiGLU epilogue (gemm_fp8_swiglu)."""
        t = ctx.torch
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.uint8)
        n, k = codes.shape
        out = np.empty(lib().dsuf_packed_bytes(FMT_FP8, MODE_MX, n, k), np.uint8)
        rc = lib().dsuf_pack_fp8_weight_gate_up(_np_ptr(codes), _np_ptr(scales), n, k, _np_ptr(out))
        if rc:
            raise DsufError(rc, "dsuf_pack_fp8_weight_gate_up")
        return Weight(ctx, FMT_FP8, MODE_MX, n, k, 1, True, t.from_numpy(out).to(ctx.device))

    @staticmethod
    def experts_fp4(ctx, codes, scales, gate_up):
        """codes u8 [E][n][k/2], scales u8 [E][n][k/32] (host arrays); gate_up: rows are [gate; up]."""
        t = ctx.torch
        e, n, kh = codes.shape
        per = lib().dsuf_packed_bytes(FMT_FP4, MODE_MX, n, kh * 2)
        tiles = t.empty(e * per, dtype=t.uint8, device=ctx.device)
        for i in range(e):
            tiles[i * per:(i + 1) * per].copy_(t.from_numpy(pack_fp4_weight(codes[i], scales[i], gate_up)))
        return Weight(ctx, FMT_FP4, MODE_MX, n, kh * 2, e, gate_up, tiles)

    @staticmethod
    def experts_fp4_packed(ctx, tiles, n, k, n_experts, gate_up):
        return Weight(ctx, FMT_FP4, MODE_MX, n, k, n_experts, gate_up, tiles)


def act_quant(ctx, mode, x, q=None, s=None):
    """tc_quant_rows (cu/tcgemm.cu:300): x bf16 [m][k] -> (codes u8 [m][k], scales)."""
    t = ctx.torch
    m, k = x.shape
    blk = 32 if mode == MODE_MX else 128
    if q is None:
        q = t.empty((m, k), dtype=t.uint8, device=x.device)
    if s is None:
        s = t.empty((m, k // blk), dtype=t.uint8 if mode == MODE_MX else t.float32, device=x.device)
    ctx.check(lib().dsuf_act_quant_fp8(ctx.h, ctx.stream(), mode, x.data_ptr(), x.stride(0), m, k, q.data_ptr(), s.data_ptr()))
    return q, s


def row_sumsq(ctx, x, out=None):
    """tc_row_sumsq (cu/tcgemm.cu:341): fp32 sum of squares of every bf16 row."""
    t = ctx.torch
    m, k = x.shape
    if out is None:
        out = t.empty(m, dtype=t.float32, device=x.device)
    ctx.check(lib().dsuf_row_sumsq(ctx.h, ctx.stream(), x.data_ptr(), x.stride(0), m, k, out.data_ptr()))
    return out


def act_quant_prenorm(ctx, mode, x, norm_w, eps, sumsq=None, q=None, s=None):
    """tc_quant_rows with RMS pre-normalisation (cu/tcgemm.cu:300): quantizes bf16(norm_w * (x * rs))."""
    t = ctx.torch
    m, k = x.shape
    blk = 32 if mode == MODE_MX else 128
    if sumsq is None:
        sumsq = row_sumsq(ctx, x)
    if q is None:
        q = t.empty((m, k), dtype=t.uint8, device=x.device)
    if s is None:
        s = t.empty((m, k // blk), dtype=t.uint8 if mode == MODE_MX else t.float32, device=x.device)
    ctx.check(lib().dsuf_act_quant_fp8_prenorm(ctx.h, ctx.stream(), mode, x.data_ptr(), x.stride(0), m, k, norm_w.data_ptr(),
                                               sumsq.data_ptr(), eps, q.data_ptr(), s.data_ptr()))
    return q, s


def gemm_fp8(ctx, w, xq, xs, m, out=None, alpha=1.0):
    t = ctx.torch
    if out is None:
        out = t.empty((m, w.n), dtype=t.bfloat16, device=xq.device)
    ctx.check(lib().dsuf_gemm_fp8(ctx.h, ctx.stream(), w.h, xq.data_ptr(), xs.data_ptr(), m, out.data_ptr(), out.stride(0),
                                  alpha, ctx.workspace.data_ptr()))
    return out


def gemm_fp8_swiglu(ctx, w, xq, xs, m, out=None, swiglu_limit=0.0):
    """The FP8 shared expert's gate/up projection (gemm_tc with Epilogue::SwiGlu, model.rs:3081-3084): w packed by
    Weight.dense_fp8_gate_up; returns bf16 [m][n/2] = silu(gate) * up."""
    t = ctx.torch
    if out is None:
        out = t.empty((m, w.n // 2), dtype=t.bfloat16, device=xq.device)
    o = GemmOpts(1.0, 0, 0, 0, 0, EPI_SWIGLU, swiglu_limit)
    ctx.check(lib().dsuf_gemm_fp8_ex(ctx.h, ctx.stream(), w.h, xq.data_ptr(), xs.data_ptr(), m, out.data_ptr(), out.stride(0), C.byref(o),
                                     ctx.workspace.data_ptr()))
    return out


def gemm_fp8_ex(ctx, w, xq, xs, m, alpha=1.0, out_f32=False, n_split=0, out=None, out2=None, sqrt_softplus=False, accumulate=False,
                rope=None):
    """dsuf_gemm_fp8_ex = ops::gemv with GemvOpts {alpha, out_f32, split} (ops.rs:165-193): fp32 or bf16 output, and with
    ``n_split`` > 0 the weight rows from n_split on go to a second tensor.  ``sqrt_softplus``: the router-gate epilogue
    (Epilogue::SqrtSoftplus), fp32 scores.  ``accumulate``: fp32 ``out`` += result (deterministic).  ``rope`` = (cos f32 [pos][32], sin, pos int32 [1] on the device,
    head, off): the fused rotary embedding of GemvOpts.rope on the first output.  Returns out, or (out, out2)."""
    t = ctx.torch
    out_f32 = out_f32 or sqrt_softplus or accumulate
    dt = t.float32 if out_f32 else t.bfloat16
    n1 = n_split if n_split > 0 else w.n
    if out is None:
        out = t.empty((m, n1), dtype=dt, device=xq.device)
    if n_split > 0 and out2 is None:
        out2 = t.empty((m, w.n - n_split), dtype=dt, device=xq.device)
    o = GemmOpts(alpha, int(bool(out_f32)), n_split, out2.stride(0) if out2 is not None else 0, out2.data_ptr() if out2 is not None else 0,
                 EPI_SQRT_SOFTPLUS if sqrt_softplus else EPI_ACCUMULATE if accumulate else EPI_STORE, 0.0)
    if rope is not None:
        cos, sin, pos, head, off = rope
        o.rope_cos, o.rope_sin, o.rope_pos, o.rope_head, o.rope_off = cos.data_ptr(), sin.data_ptr(), pos.data_ptr(), int(head), int(off)
    ctx.check(lib().dsuf_gemm_fp8_ex(ctx.h, ctx.stream(), w.h, xq.data_ptr(), xs.data_ptr(), m, out.data_ptr(), out.stride(0), C.byref(o),
                                     ctx.workspace.data_ptr()))
    return (out, out2) if n_split > 0 else out


def gemm_fp8_static(ctx, w, xq, xs, m, out=None, alpha=1.0):
    """dsuf_gemm_fp8 without a caller workspace (scratch is a fixed array inside the library); see include/dsuf_qmm.h."""
    t = ctx.torch
    if out is None:
        out = t.empty((m, w.n), dtype=t.bfloat16, device=xq.device)
    ctx.check(lib().dsuf_gemm_fp8_static(ctx.h, ctx.stream(), w.h, xq.data_ptr(), xs.data_ptr(), m, out.data_ptr(), out.stride(0),
                                         alpha))
    return out


def gemv(ctx, w, x, out=None, alpha=1.0):
    """ops::gemv (ops.rs:331-474): bf16 activations in, bf16 out; quantizes once, then streams the weight."""
    xq, xs = act_quant(ctx, w.mode, x)
    return gemm_fp8(ctx, w, xq, xs, x.shape[0], out, alpha)


class PeerAllReduce:
    """dsuf_ep_allreduce_bf16 over buffers that every rank of a torch.distributed group has mapped (torch symmetric memory).

    ``buffer(shape)`` hands out bf16 partial buffers in symmetric memory (the kernels that produce a partial write
    straight into them); ``__call__(partial, out)`` sums that buffer over the ranks into the local tensor ``out``."""

    def __init__(self, ctx, dist, rank, world):
        import torch.distributed._symmetric_memory as symm
        self.ctx, self.rank, self.world, self.symm = ctx, rank, world, symm
        self.group = dist.group.WORLD.group_name
        t = ctx.torch
        nflag = lib().dsuf_ep_flag_bytes(world) // 4
        self.flags = symm.empty(nflag, dtype=t.int32, device=ctx.device)
        self.flags.zero_()
        h = symm.rendezvous(self.flags, self.group)
        self.flag_ptrs = (C.c_uint64 * world)(*[int(p) for p in h.buffer_ptrs])
        self.state = t.zeros(2, dtype=t.int32, device=ctx.device)
        self.data_ptrs = {}
        self.stages = {}
        t.cuda.synchronize()
        dist.barrier()   # every rank's flag block is zero before anyone announces

    def buffer(self, shape):
        t = self.ctx.torch
        buf = self.symm.empty(*shape, dtype=t.bfloat16, device=self.ctx.device)
        h = self.symm.rendezvous(buf, self.group)
        self.data_ptrs[buf.data_ptr()] = (C.c_uint64 * self.world)(*[int(p) for p in h.buffer_ptrs])
        return buf

    TWO_SHOT_BYTES = 8 << 20   # from here on a rank sums only its own 1/W of the elements and the sums are gathered

    def __call__(self, partial, out):
        ptrs = self.data_ptrs[partial.data_ptr()]
        n = partial.numel()
        stage = self.stages.get(partial.data_ptr())
        if stage is not None and n * 2 >= self.TWO_SHOT_BYTES and n % (8 * self.world) == 0:
            # Large messages (prefill-size batches): reduce-scatter + all-gather with the same two kernels.  Rank r sums
            # elements [r n/W, (r+1) n/W) of every partial into its slice of `stage` (a second mapped buffer), then every
            # rank gathers the slices: 2 (W-1)/W n elements pulled per rank instead of (W-1) n -- the large-M shape of the
            # reference's comm_push2 (crates/kernels/cu/comm.cu:323-542).
            sl = n // self.world
            off = self.rank * sl * 2
            sub = (C.c_uint64 * self.world)(*[int(p) + off for p in ptrs])
            self.ctx.check(lib().dsuf_ep_allreduce_bf16(self.ctx.h, self.ctx.stream(), sub, self.flag_ptrs, self.rank, self.world, sl,
                                                        self.state.data_ptr(), stage.data_ptr() + off))
            sptrs = self.data_ptrs[stage.data_ptr()]
            self.ctx.check(lib().dsuf_ep_allgather_cols_bf16(self.ctx.h, self.ctx.stream(), sptrs, self.flag_ptrs, self.rank, self.world,
                                                             1, n, self.state.data_ptr(), out.data_ptr()))
            return out
        self.ctx.check(lib().dsuf_ep_allreduce_bf16(self.ctx.h, self.ctx.stream(), ptrs, self.flag_ptrs, self.rank, self.world,
                                                    n, self.state.data_ptr(), out.data_ptr()))
        return out

    def stage_for(self, partial):
        """Registers a second mapped buffer of the same shape for the two-shot all-reduce of ``partial``."""
        self.stages[partial.data_ptr()] = self.buffer(tuple(partial.shape))

    def gather_cols(self, buf, out):
        """dsuf_ep_allgather_cols_bf16: every rank wrote its column slice of ``buf`` (a buffer from ``buffer``); ``out``
        receives all slices."""
        rows, cols = buf.shape
        ptrs = self.data_ptrs[buf.data_ptr()]
        self.ctx.check(lib().dsuf_ep_allgather_cols_bf16(self.ctx.h, self.ctx.stream(), ptrs, self.flag_ptrs, self.rank, self.world,
                                                         rows, cols, self.state.data_ptr(), out.data_ptr()))
        return out

    def combine(self, plan, yrows, shared, partial, out, quant=None):
        """dsuf_ep_combine_bf16: the local sum of every token's expert rows and its exchange in one kernel.
        ``quant`` = (mode, xq, xs): also leave ``out`` quantized for the next projection (dsuf_ep_combine_quant_bf16)."""
        tok, h = out.shape
        ptrs = self.data_ptrs[partial.data_ptr()]
        mode, xq, xs = quant if quant is not None else (MODE_DS, None, None)
        self.ctx.check(lib().dsuf_ep_combine_quant_bf16(self.ctx.h, self.ctx.stream(), plan.pair_row.data_ptr(), yrows.data_ptr(),
                                                        shared.data_ptr() if shared is not None else 0, tok, plan.topk, h, ptrs,
                                                        self.flag_ptrs, self.rank, self.world, self.state.data_ptr(), out.data_ptr(),
                                                        mode, xq.data_ptr() if xq is not None else 0, xs.data_ptr() if xs is not None else 0))
        return out


def lm_head(ctx, w, x, alpha=1.0, out=None, temperature=None, valid_rows=0, id_offset=0, records=None):
    """dsuf_lm_head_bf16 = the output head, ops::gemv with GemvOpts {persist, out_f32, samp_rec} (crates/engine/src/ops.rs:165-193):
    fp32 logits [m][n] of bf16 token rows x [m][k] (m <= 16) against the row-major bf16 weight w [n][k].  With a
    ``temperature`` the per-quad sampling records float [m][n/64][20] are written too; returns (logits, records)."""
    t = ctx.torch
    n, k = w.shape
    m = x.shape[0]
    if out is None:
        out = t.empty((m, n), dtype=t.float32, device=x.device)
    sp = None
    if temperature is not None:
        if records is None:
            records = t.zeros((m, n // 64, 20), dtype=t.float32, device=x.device)
        sp = SamplingOpts(records.data_ptr(), float(temperature), int(valid_rows), int(id_offset))
    ctx.check(lib().dsuf_lm_head_bf16(ctx.h, ctx.stream(), w.data_ptr(), n, k, x.data_ptr(), x.stride(0), m, alpha, out.data_ptr(),
                                      out.stride(0), C.byref(sp) if sp is not None else None))
    return (out, records) if temperature is not None else out


def probe_tensor_rate(ctx, n_cols=128, a_is_e2m1=False, iters=20000, reps=5):
    """TFLOP/s the tensor cores deliver to the library's MMA instruction with no memory traffic (dsuf_probe_tensor_rate),
    best of ``reps`` launches timed with CUDA events."""
    t = ctx.torch
    flop = C.c_double()
    best = 0.0
    for _ in range(reps + 1):
        e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
        e0.record()
        ctx.check(lib().dsuf_probe_tensor_rate(ctx.h, ctx.stream(), n_cols, int(bool(a_is_e2m1)), iters, C.byref(flop)))
        e1.record()
        t.cuda.synchronize()
        best = max(best, flop.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


class MoePlan:
    """Caller-owned buffers of the permute plan (MpParams, ops.rs:1478-1491)."""

    def __init__(self, ctx, tokens, topk, n_exp, tile_rows):
        t = ctx.torch
        dev = ctx.device
        self.ctx, self.tokens, self.topk, self.n_exp, self.tile_rows = ctx, tokens, topk, n_exp, tile_rows
        p = tokens * topk
        self.p = p
        self.max_tiles = p // tile_rows + n_exp
        i32 = dict(dtype=t.int32, device=dev)
        self.expert_off = t.zeros(n_exp + 1, **i32)
        self.row_pair = t.zeros(max(p, 1), **i32)
        self.pair_row = t.zeros(max(p, 1), **i32)
        self.row_w = t.zeros(max(p, 1), dtype=t.float32, device=dev)
        self.tiles = t.zeros((self.max_tiles, 4), **i32)
        self.ntiles = t.zeros(2, **i32)
        self.scratch = t.zeros(lib().dsuf_moe_plan_scratch_ints(p, n_exp), **i32)
        self.c = PlanStruct(self.expert_off.data_ptr(), self.row_pair.data_ptr(), self.pair_row.data_ptr(),
                            self.row_w.data_ptr(), self.tiles.data_ptr(), self.ntiles.data_ptr(), self.scratch.data_ptr(),
                            p, n_exp, tile_rows, self.max_tiles)


def moe_route_tokens(ctx, score_fn, scores, bias, topk, route_scale=1.0, ids=None, w=None):
    t = ctx.torch
    tok, n_exp = scores.shape
    if ids is None:
        ids = t.empty((tok, topk), dtype=t.int32, device=scores.device)
    if w is None:
        w = t.empty((tok, topk), dtype=t.float32, device=scores.device)
    ctx.check(lib().dsuf_moe_route(ctx.h, ctx.stream(), score_fn, scores.data_ptr(), bias.data_ptr() if bias is not None else 0,
                                   tok, n_exp, topk, route_scale, ids.data_ptr(), w.data_ptr()))
    return ids, w


def moe_perm(ctx, plan, ids, w, e_lo=0):
    ctx.check(lib().dsuf_moe_permute_plan(ctx.h, ctx.stream(), ids.data_ptr(), w.data_ptr(), e_lo, C.byref(plan.c)))


def moe_gather_quant(ctx, mode, plan, x, xq, xs):
    tok, h = x.shape
    ctx.check(lib().dsuf_moe_gather_quant(ctx.h, ctx.stream(), mode, x.data_ptr(), x.stride(0), tok, h, plan.topk,
                                          C.byref(plan.c), xq.data_ptr(), xs.data_ptr()))


def moe_route_plan_gather(ctx, score_fn, scores, bias, topk, route_scale, ids, w, e_lo, plan, mode, x, xq, xs):
    """dsuf_moe_route_plan_gather: router + permute plan + gather/quant of a decode-size batch in one launch."""
    tok, h = x.shape
    ctx.check(lib().dsuf_moe_route_plan_gather(ctx.h, ctx.stream(), score_fn, scores.data_ptr(), bias.data_ptr() if bias is not None else 0,
                                               tok, scores.shape[1], topk, route_scale, ids.data_ptr(), w.data_ptr(), e_lo, C.byref(plan.c),
                                               mode, x.data_ptr(), x.stride(0), h, xq.data_ptr(), xs.data_ptr()))


def moe_gather_quant_prenorm(ctx, mode, plan, x, norm_w, eps, xq, xs, sumsq=None):
    """moe_gather_quant with RMS pre-normalisation (cu/tcmoe.cu:88): bf16(norm_w * (x * rs)) quantised once per token."""
    tok, h = x.shape
    if sumsq is None:
        sumsq = row_sumsq(ctx, x)
    ctx.check(lib().dsuf_moe_gather_quant_prenorm(ctx.h, ctx.stream(), mode, x.data_ptr(), x.stride(0), tok, h, plan.topk,
                                                  C.byref(plan.c), norm_w.data_ptr(), sumsq.data_ptr(), eps, xq.data_ptr(), xs.data_ptr()))


def moe_w13_swiglu(ctx, w13, act_mode, plan, xq, xs, act_out, swiglu_limit=0.0):
    ctx.check(lib().dsuf_moe_w13_swiglu(ctx.h, ctx.stream(), w13.h, act_mode, C.byref(plan.c), xq.data_ptr(), xs.data_ptr(),
                                        swiglu_limit, act_out.data_ptr()))


def moe_w2(ctx, w2, act_mode, plan, act_q, act_s, yrows):
    ctx.check(lib().dsuf_moe_w2(ctx.h, ctx.stream(), w2.h, act_mode, C.byref(plan.c), act_q.data_ptr(), act_s.data_ptr(),
                                yrows.data_ptr()))


def moe_unpermute(ctx, plan, yrows, out, shared=None, quant=None):
    """dsuf_moe_unpermute; with ``quant`` = (mode, xq, xs) the result is also left quantized for the next projection
    (dsuf_moe_unpermute_quant: codes and scales of act_quant(out), bit for bit)."""
    tok, h = out.shape
    sh = shared.data_ptr() if shared is not None else 0
    if quant is not None:
        mode, xq, xs = quant
        ctx.check(lib().dsuf_moe_unpermute_quant(ctx.h, ctx.stream(), C.byref(plan.c), yrows.data_ptr(), sh, tok, plan.topk, h,
                                                 out.data_ptr(), out.stride(0), mode, xq.data_ptr(), xs.data_ptr()))
        return
    ctx.check(lib().dsuf_moe_unpermute(ctx.h, ctx.stream(), C.byref(plan.c), yrows.data_ptr(), sh, tok, plan.topk, h, out.data_ptr(),
                                       out.stride(0)))


class MoeLayer:
    """Routed-expert FFN of one layer = Rank::ffn / ffn_prefill (crates/engine/src/model.rs:3497, :3063) without the
    model-specific parts: route -> plan -> gather+quant -> w13+SwiGLU -> quant -> w2 -> unpermute/combine.
    All scratch is allocated once here; ``forward`` only launches kernels."""

    def __init__(self, ctx, w13, w2, tokens, topk, act_mode, e_lo=0, tile_rows=None, swiglu_limit=0.0):
        t = ctx.torch
        dev = ctx.device
        self.ctx, self.w13, self.w2, self.tokens, self.topk, self.act_mode = ctx, w13, w2, tokens, topk, act_mode
        self.e_lo, self.swiglu_limit = e_lo, swiglu_limit
        self.fuse_front = True   # decode-size batches: router + plan + gather/quant in one launch (when forward gets `route`)
        self.h, self.inter = w13.k, w13.n // 2
        if tile_rows is None:
            tile_rows = 8
        self.plan = MoePlan(ctx, tokens, topk, w13.n_experts, tile_rows)
        p = max(tokens * topk, 1)
        blk = 32 if act_mode == MODE_MX else 128
        sdt = t.uint8 if act_mode == MODE_MX else t.float32
        self.xq = t.zeros((p, self.h), dtype=t.uint8, device=dev)
        self.xs = t.zeros((p, self.h // blk), dtype=sdt, device=dev)
        self.act = t.zeros((p, self.inter), dtype=t.bfloat16, device=dev)
        self.act_q = t.zeros((p, self.inter), dtype=t.uint8, device=dev)
        self.act_s = t.zeros((p, self.inter // blk), dtype=sdt, device=dev)
        self.yrows = t.zeros((p, self.h), dtype=t.float32, device=dev)

    def forward(self, x, ids, w, out, shared=None, events=None, combine=None, route=None, out_quant=None):
        """``events``: optional list; (start, end) CUDA events around the gate/up kernel are appended (bench timing).
        ``combine``: optional callable (plan, yrows, shared) -> tensor that replaces the local unpermute (the
        expert-parallel stack passes the kernel that sums locally and across ranks in one launch).
        ``route``: optional (score_fn, scores [t][experts], bias, route_scale): the router runs here and writes ``ids`` / ``w``;
        decode-size batches (at most 1024 pairs) take one launch for router + plan + gather/quant.
        ``out_quant``: optional (mode, xq, xs): the unpermute also leaves ``out`` quantized for the next projection."""
        ctx, plan = self.ctx, self.plan
        if events is None:
            events = getattr(self, "events", None)
        if route is not None and plan.p <= 1024 and plan.p > 0 and self.fuse_front:
            score_fn, scores, bias, scale = route
            moe_route_plan_gather(ctx, score_fn, scores, bias, self.topk, scale, ids, w, self.e_lo, plan, self.act_mode, x, self.xq, self.xs)
        else:
            if route is not None:
                score_fn, scores, bias, scale = route
                moe_route_tokens(ctx, score_fn, scores, bias, self.topk, scale, ids=ids, w=w)
            moe_perm(ctx, plan, ids, w, self.e_lo)
            moe_gather_quant(ctx, self.act_mode, plan, x, self.xq, self.xs)
        if events is not None:
            # inside a stream capture the events must be recorded as graph nodes of their own (external events), so that
            # every replay of the graph stamps them
            ext = {"external": True} if ctx.torch.cuda.is_current_stream_capturing() else {}
            e0, e1 = ctx.torch.cuda.Event(enable_timing=True, **ext), ctx.torch.cuda.Event(enable_timing=True, **ext)
            e0.record()
        moe_w13_swiglu(ctx, self.w13, self.act_mode, plan, self.xq, self.xs, self.act, self.swiglu_limit)
        if events is not None:
            e1.record()
            events.append((e0, e1))
        act_quant(ctx, self.act_mode, self.act, self.act_q, self.act_s)
        moe_w2(ctx, self.w2, self.act_mode, plan, self.act_q, self.act_s, self.yrows)
        if combine is not None:
            return combine(plan, self.yrows, shared)
        moe_unpermute(ctx, plan, self.yrows, out, shared, quant=out_quant)
        return out
