"""The REFERENCE's own sm_100a kernels, launched on the GPU: the second, independent checker next to the CPU restatement.

Test and benchmark infrastructure only (as everything under oracle/): the product never imports it.

``make -C oracle ref_cubins`` compiles the reference's .cu files, where they lie, into ``oracle/_ref/*.cubin`` with the
flags of crates/kernels/build.rs:42-43; ``oracle/librefk.so`` (refk.cc) loads a cubin and launches a kernel by name the
way crates/cuda/src/lib.rs:630-664 does.  This module restates, per kernel, what the reference's Rust host code decides:
the ``#[repr(C)]`` parameter struct, the grid / block / cluster / shared-memory arithmetic, the tensor maps and the host
weight layouts -- each function cites the lines it follows.  Preconditions the Rust code checks with ``ensure!`` are
checked here BEFORE anything is launched: the reference's device-side waits are unbounded, so a launch whose geometry is
wrong must never reach the GPU.  Only kernels whose waits are on CTA-local (or cluster-local) mbarriers are offered;
kernels that spin on global memory written by other CTAs or other GPUs (comm.cu, the fused decode MoE) are left out.

Arguments are torch CUDA tensors; launches go to torch's current stream.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
LIB_PATH = os.path.join(HERE, "librefk.so")

_LIB = None
_MODULES = {}
_FUNCS = {}
_TMAPS = {}  # uploaded tensor maps by (base, dims, box)
_KEEP = []   # host-side parameter blocks of launches in flight are kept alive until the next synchronize()


class RefKernelError(RuntimeError):
    pass


def available():
    """True when the launcher library and at least the cubins used here have been built."""
    return os.path.exists(LIB_PATH) and all(os.path.exists(os.path.join(REF_DIR, f + ".cubin")) for f in ("tcgemm", "tcmoe", "ops"))


def lib():
    global _LIB
    if _LIB is None:
        L = C.CDLL(LIB_PATH)
        L.refk_last_error.restype = C.c_char_p
        L.refk_load.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        L.refk_function.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]
        L.refk_set_smem.argtypes = [C.c_void_p, C.c_int]
        L.refk_allow_big_cluster.argtypes = [C.c_void_p]
        L.refk_func_attr.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int)]
        L.refk_launch.argtypes = [C.c_void_p] + [C.c_uint] * 10 + [C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]
        L.refk_tmap_u8_sw128.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32]
        L.refk_tmap_fp4_rows.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint32]
        L.refk_tmap_fp4_unpack_strided.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32]
        _LIB = L
    return _LIB


def _check(rc):
    if rc:
        raise RefKernelError(lib().refk_last_error().decode())


def require(cond, msg):
    """The reference's ``ensure!``: a launch contract that does not hold stops here, on the host."""
    if not cond:
        raise RefKernelError("precondition: " + msg)


def function(cubin, name, smem=0, big_cluster=False):
    """Kernels::get (crates/kernels/src/lib.rs:47-49) + Function::set_max_dynamic_smem."""
    key = (cubin, name)
    if key not in _FUNCS:
        if cubin not in _MODULES:
            m = C.c_void_p()
            _check(lib().refk_load(os.path.join(REF_DIR, cubin + ".cubin").encode(), C.byref(m)))
            _MODULES[cubin] = m
        f = C.c_void_p()
        _check(lib().refk_function(_MODULES[cubin], name.encode(), C.byref(f)))
        _FUNCS[key] = [f, 0, False]
    ent = _FUNCS[key]
    if smem > ent[1]:
        require(smem <= 232448, f"{name}: {smem} bytes of dynamic shared memory exceed the 227 KB opt-in")
        _check(lib().refk_set_smem(ent[0], smem))
        ent[1] = smem
    if big_cluster and not ent[2]:
        _check(lib().refk_allow_big_cluster(ent[0]))
        ent[2] = True
    return ent[0]


def launch(fn, grid, block, smem, args, cluster=(1, 1, 1), pdl=False):
    """cu::launch (crates/cuda/src/lib.rs:630-664).  ``args``: ctypes objects, one per kernel parameter."""
    import torch
    g = tuple(grid) + (1,) * (3 - len(grid))
    b = (block, 1, 1) if isinstance(block, int) else tuple(block) + (1,) * (3 - len(block))
    require(all(x >= 1 for x in g + b), "empty grid or block")
    require(g[0] % cluster[0] == 0 and g[1] % cluster[1] == 0 and g[2] % cluster[2] == 0, "grid not a multiple of the cluster")
    arr = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
    _KEEP.append((args, arr))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _check(lib().refk_launch(fn, g[0], g[1], g[2], b[0], b[1], b[2], smem, cluster[0], cluster[1], cluster[2], int(pdl), stream, arr))


def synchronize():
    import torch
    torch.cuda.synchronize()
    _KEEP.clear()


def upload_tmap_u8_sw128(base_tensor, cols, rows, stride, box_rows):
    """tensor_map_u8_sw128 (crates/cuda/src/lib.rs:742-763) uploaded to device memory (cu::upload_synced)."""
    import torch
    require(base_tensor.data_ptr() % 16 == 0 and stride % 16 == 0 and box_rows <= 256, "tensor map alignment / box")
    key = (base_tensor.data_ptr(), cols, rows, stride, box_rows)
    if key in _TMAPS:                  # the reference caches its activation maps the same way (model.rs:1343-1358)
        return _TMAPS[key]
    host = np.zeros(128, np.uint8)
    _check(lib().refk_tmap_u8_sw128(host.ctypes.data_as(C.c_void_p), base_tensor.data_ptr(), cols, rows, stride, box_rows))
    dev = torch.from_numpy(host).cuda()
    require(dev.data_ptr() % 64 == 0, "tensor map must be 64-byte aligned in device memory")
    _TMAPS[key] = dev
    return dev


# ------------------------------------------------------------------------------------------------ host layouts
def sf_atoms(scales_rows):
    """tile_sf_blocks (crates/model/src/formats.rs:216-228): UE8M0 scales u8 [n][k/32] (one per row and 32-K block) ->
    512-byte tcgen05 scale-factor atoms ordered [n/128][k/128]: byte (r%32)*16 + (r%128/32)*4 + kb%4."""
    s = np.ascontiguousarray(scales_rows, dtype=np.uint8)
    n, kb = s.shape
    require(n % 128 == 0 and kb % 4 == 0, "tile_sf_blocks needs n % 128 == 0 and k % 128 == 0")
    rt, kt = n // 128, kb // 4
    a = s.reshape(rt, 4, 32, kt, 4).transpose(0, 3, 2, 1, 4)   # [rt][kt][r%32][r/32][kb%4]
    return np.ascontiguousarray(a).reshape(rt * kt * 512)


def sf_atoms_to_rows(atoms, n, k):
    """Inverse of sf_atoms: [n/128][k/128][512] -> u8 [n][k/32]."""
    rt, kt = n // 128, k // 128
    a = np.asarray(atoms, dtype=np.uint8).reshape(rt, kt, 32, 4, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(a).reshape(n, k // 32)


def kpos32(k):
    """crates/kernels/cu/common.cuh:67: position of element k inside its 32-K block in the mma.sync B-fragment order."""
    return 8 * ((k & 7) >> 1) + (k & 1) + 2 * ((k >> 3) & 1) + 4 * (k >> 4)


class TcWeight:
    """Loader::tc_copy (crates/engine/src/weights.rs:181-214): the tcgen05-side image of a dense FP8 weight -- row-major
    codes, the 32x32 UE8M0 scales expanded per row into scale-factor atoms, and tensor maps with 128- and nt-row boxes."""

    def __init__(self, codes, scales32):
        import torch
        codes = np.ascontiguousarray(codes, np.uint8)
        n, k = codes.shape
        require(n % 128 == 0 and k % 128 == 0, "this harness takes n % 128 == 0 and k % 128 == 0 (tc_copy pads K; not needed here)")
        self.n, self.k = n, k
        self.nt = 256 if n % 256 == 0 else 128
        s_rows = np.repeat(np.asarray(scales32, np.uint8).reshape(n // 32, k // 32), 32, axis=0)
        self.w = torch.from_numpy(codes).cuda()
        self.sf = torch.from_numpy(sf_atoms(s_rows)).cuda()
        self.tmap = upload_tmap_u8_sw128(self.w, k, n, k, self.nt)
        self.tmap128 = self.tmap if self.nt == 128 else upload_tmap_u8_sw128(self.w, k, n, k, 128)


# ------------------------------------------------------------------------------------------------ parameter structs
class TqParams(C.Structure):      # crates/engine/src/ops.rs:1571-1583, cu/tcgemm.cu:289-298
    _fields_ = [("x", C.c_uint64), ("ldx", C.c_int32), ("m", C.c_int32), ("k", C.c_int32), ("_pad", C.c_int32), ("pw", C.c_uint64),
                ("norm_part", C.c_uint64), ("nslices", C.c_int32), ("eps", C.c_float), ("aq", C.c_uint64), ("sfa", C.c_uint64)]


class TgParams(C.Structure):      # crates/engine/src/ops.rs:1548-1568, cu/tcgemm.cu:3-16
    _fields_ = [("ta", C.c_uint64), ("tb", C.c_uint64), ("sfa", C.c_uint64), ("sfb", C.c_uint64), ("out", C.c_uint64), ("ldo", C.c_int32),
                ("out_f32", C.c_int32), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("nt", C.c_int32), ("alpha", C.c_float),
                ("_pad", C.c_int32), ("out2", C.c_uint64), ("ldo2", C.c_int32), ("n_split", C.c_int32), ("swiglu", C.c_int32),
                ("swiglu_limit", C.c_float)]


class MpParams(C.Structure):      # crates/engine/src/ops.rs:1478-1491, cu/tcmoe.cu:6-16
    _fields_ = [("ids", C.c_uint64), ("w", C.c_uint64), ("m", C.c_int32), ("topk", C.c_int32), ("n_exp", C.c_int32), ("_pad", C.c_int32),
                ("row_pair", C.c_uint64), ("row_w", C.c_uint64), ("pair_row", C.c_uint64), ("row_tile", C.c_uint64), ("tiles", C.c_uint64),
                ("ntiles", C.c_uint64)]


class MqParams(C.Structure):      # crates/engine/src/ops.rs:1495-1509, cu/tcmoe.cu:71-82
    _fields_ = [("x", C.c_uint64), ("ldx", C.c_int32), ("m", C.c_int32), ("k", C.c_int32), ("topk", C.c_int32), ("pw", C.c_uint64),
                ("norm_part", C.c_uint64), ("nslices", C.c_int32), ("eps", C.c_float), ("pair_row", C.c_uint64), ("row_tile", C.c_uint64),
                ("xq", C.c_uint64), ("sf", C.c_uint64)]


assert C.sizeof(TqParams) == 64 and C.sizeof(TgParams) == 96 and C.sizeof(MpParams) == 80 and C.sizeof(MqParams) == 80

TGP_SMEM = 6 * 34816 + 1024       # crates/engine/src/ops.rs:1585


def tg_smem(nt):                  # crates/engine/src/ops.rs:1587-1590
    sb = (16384 + nt * 128 + 512 + max(nt // 128, 1) * 512 + 1023) & ~1023
    return 4 * sb + 1024


def sm_count():
    import torch
    return torch.cuda.get_device_properties(0).multi_processor_count


# ------------------------------------------------------------------------------------------------ kernels
def tc_row_sumsq(x):
    """tc_row_sumsq (cu/tcgemm.cu:342-356, launched by Rank::gemm_tc, model.rs:1335): part f32 [m][26], the row's sum of
    squares at index 25."""
    import torch
    m, k = x.shape
    require(x.dtype == torch.bfloat16 and x.stride(1) == 1 and k % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0, "bf16 rows, 16-byte aligned")
    part = torch.zeros(m, 26, dtype=torch.float32, device=x.device)
    f = function("tcgemm", "tc_row_sumsq")
    launch(f, ((m + 7) // 8,), 256, 0, [C.c_uint64(x.data_ptr()), C.c_int32(x.stride(0)), C.c_int32(m), C.c_int32(k), C.c_uint64(part.data_ptr())])
    return part


def tc_quant_rows(x, pw=None, eps=0.0, part=None, rows_alloc=None, aq=None, sfa=None):
    """tc_quant_rows (cu/tcgemm.cu:300-340) as Rank::gemm_tc launches it (model.rs:1328-1345): one CTA per row,
    min(ceil(k/32 / 32) * 32, 256) threads.  Returns (aq u8 [rows_alloc][k], sfa atoms u8 [rows_alloc/128 * k/128 * 512])."""
    import torch
    m, k = x.shape
    require(x.dtype == torch.bfloat16 and x.stride(1) == 1 and k % 128 == 0, "k % 128 == 0 (model.rs:1331)")
    require(x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0, "16-byte aligned rows")
    rows_alloc = rows_alloc or (m + 127) // 128 * 128
    require(rows_alloc >= m and rows_alloc % 128 == 0, "scratch rows")
    if aq is None:
        aq = torch.zeros(rows_alloc, k, dtype=torch.uint8, device=x.device)
        sfa = torch.full((rows_alloc // 128 * (k // 128) * 512,), 127, dtype=torch.uint8, device=x.device)
    require(aq.shape == (rows_alloc, k) and sfa.numel() == rows_alloc // 128 * (k // 128) * 512, "scratch sizes")
    if pw is not None:
        require(pw.dtype == torch.bfloat16 and pw.numel() == k and pw.data_ptr() % 16 == 0, "norm weight bf16 [k]")
        if part is None:
            part = tc_row_sumsq(x)
    p = TqParams(x.data_ptr(), x.stride(0), m, k, 0, pw.data_ptr() if pw is not None else 0, part.data_ptr() if pw is not None else 0,
                 1 if pw is not None else 0, float(eps), aq.data_ptr(), sfa.data_ptr())
    threads = min(((k // 32) + 31) // 32 * 32, 256)
    launch(function("tcgemm", "tc_quant_rows"), (m,), threads, 0, [p])
    _KEEP.append((x, pw, part))
    return aq, sfa


def tc_gemm(tw, aq, sfa, m, out=None, alpha=1.0, persistent=None, out_f32=False):
    """The prefill dense GEMM as Rank::gemm_tc picks it (model.rs:1359-1369): tc_gemm_fp8p (persistent, 128-column tiles,
    grid min(tiles, SMs) x 256 threads, TGP_SMEM) unless the one-tile-per-CTA grid of tc_gemm_fp8 (grid (n/nt, ceil(m/128)) x
    128 threads, tg_smem(nt)) fills between 2/3 and all of the SMs.  ``persistent`` forces one of the two.
    aq u8 [rows][k] and sfa atoms come from tc_quant_rows; the activation map has 128-row boxes (model.rs:1351)."""
    import torch
    n, k = tw.n, tw.k
    require(aq.shape[1] == k and aq.shape[0] % 128 == 0 and aq.shape[0] >= m and m >= 1, "activation image")
    require(sfa.numel() >= (aq.shape[0] // 128) * (k // 128) * 512, "activation scale atoms")
    if out is None:
        out = torch.empty(m, n, dtype=torch.float32 if out_f32 else torch.bfloat16, device=aq.device)
    require(out.stride(1) == 1 and out.stride(0) >= n and out.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0, "output rows 16-byte aligned")
    ta = upload_tmap_u8_sw128(aq, k, aq.shape[0], k, 128)
    sms = sm_count()
    gx, mt = n // tw.nt, (m + 127) // 128
    if persistent is None:
        persistent = not (gx * mt >= sms * 2 // 3 and gx * mt <= sms)
    gp = TgParams(ta.data_ptr(), 0, sfa.data_ptr(), tw.sf.data_ptr(), out.data_ptr(), out.stride(0), int(out_f32), m, n, k, tw.nt, float(alpha), 0,
                  0, 0, n, 0, 0.0)
    if persistent:
        require((m + 127) // 128 <= 255 and k // 128 <= 255, "tc_gemm_fp8p packs (stage, m tile, k tile) of its first loads into 8-bit fields (cu/tcgemm.cu:175,181)")
        gp.tb = tw.tmap128.data_ptr()
        tiles = (n // 128) * mt
        # expect_tx per stage = 16384 (A) + 128*128 (B) + 512 + 512 = the bytes of the two 128 x 128 boxes and two atoms
        launch(function("tcgemm", "tc_gemm_fp8p", TGP_SMEM), (min(tiles, sms),), 256, TGP_SMEM, [gp])
    else:
        gp.tb = tw.tmap.data_ptr()
        smem = tg_smem(tw.nt)
        launch(function("tcgemm", "tc_gemm_fp8", smem), (gx, mt), 128, smem, [gp])
    _KEEP.append((ta, aq, sfa, tw, out))
    return out


def moe_route_tokens(scores, bias, topk, route_scale=1.0):
    """moe_route_tokens (cu/ops.cu:615-623), launched by Rank::ffn_prefill (model.rs:3103): grid ceil(m/8) x 256 threads.
    scores f32 [m][n_exp] are the activated scores (the gate GEMV's epilogue applied sqrt-softplus); top-k of score + bias."""
    import torch
    m, n_exp = scores.shape
    require(scores.dtype == torch.float32 and scores.is_contiguous() and bias.dtype == torch.float32 and bias.numel() == n_exp, "f32 scores / bias")
    require(n_exp <= 384 and 1 <= topk <= 8, "route_token holds 12 experts per lane and moe_route_tokens 8 picks per token (cu/route.cuh:8, cu/ops.cu:619)")
    ids = torch.zeros(m, topk, dtype=torch.int32, device=scores.device)
    w = torch.zeros(m, topk, dtype=torch.float32, device=scores.device)
    launch(function("ops", "moe_route_tokens"), ((m + 7) // 8,), 256, 0,
           [C.c_int32(m), C.c_uint64(scores.data_ptr()), C.c_uint64(bias.data_ptr()), C.c_int32(n_exp), C.c_int32(topk), C.c_float(route_scale),
            C.c_uint64(ids.data_ptr()), C.c_uint64(w.data_ptr())])
    _KEEP.append((scores, bias))
    return ids, w


class PrefillPlan:
    """Buffers of MpParams (Rank::new's PrefillMoe, model.rs:854-895) and moe_perm's launch (model.rs:3106-3107)."""

    def __init__(self, ids, w, n_exp):
        import torch
        m, topk = ids.shape
        p = m * topk
        require(ids.dtype == torch.int32 and w.dtype == torch.float32 and ids.is_contiguous() and w.is_contiguous(), "ids i32, w f32")
        require(n_exp <= 512, "moe_perm keeps 512 counters (cu/tcmoe.cu:20)")
        require(p // 128 + n_exp <= 1024, "the tile list holds 1024 tiles (cu/tcmoe.cu:4, model.rs:858)")
        require(p > 0 and int(ids.min()) >= 0 and int(ids.max()) < n_exp, "expert ids outside [0, n_exp) would index past moe_perm's counters")
        dev = ids.device
        self.m, self.topk, self.n_exp, self.p = m, topk, n_exp, p
        self.row_pair = torch.zeros(p, dtype=torch.int32, device=dev)
        self.row_w = torch.zeros(p, dtype=torch.float32, device=dev)
        self.pair_row = torch.zeros(p, dtype=torch.int32, device=dev)
        self.row_tile = torch.zeros(p, dtype=torch.int32, device=dev)
        self.tiles = torch.zeros(1024, 4, dtype=torch.int32, device=dev)
        self.ntiles = torch.zeros(1, dtype=torch.int32, device=dev)
        mp = MpParams(ids.data_ptr(), w.data_ptr(), m, topk, n_exp, 0, self.row_pair.data_ptr(), self.row_w.data_ptr(), self.pair_row.data_ptr(),
                      self.row_tile.data_ptr(), self.tiles.data_ptr(), self.ntiles.data_ptr())
        launch(function("tcmoe", "moe_perm"), (1,), 1024, 0, [mp])
        _KEEP.append((ids, w))


def moe_gather_quant(x, pw, eps, plan, part=None):
    """moe_gather_quant (cu/tcmoe.cu:88-133) as Rank::ffn_prefill launches it (model.rs:3108-3124): RMS pre-normalisation
    (always on: the kernel reads pw unconditionally), 1x32 FP8 quant, every token row written to its topk permuted rows with
    the codes of each 32-K block in kpos32 order, scales into the atoms of the row's tile.  grid ceil(m*k/32 / 256) x 256."""
    import torch
    m, k = x.shape
    require(m == plan.m and k % 128 == 0 and x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.data_ptr() % 16 == 0, "bf16 [m][k], k % 128 == 0")
    require(pw is not None and pw.dtype == torch.bfloat16 and pw.numel() == k and pw.data_ptr() % 16 == 0, "moe_gather_quant needs the norm weight")
    if part is None:
        part = tc_row_sumsq(x)
    ntile_cap = plan.p // 128 + plan.n_exp
    xq = torch.zeros(plan.p + 128, k, dtype=torch.uint8, device=x.device)
    sf = torch.full((ntile_cap * (k // 128) * 512,), 127, dtype=torch.uint8, device=x.device)
    mq = MqParams(x.data_ptr(), x.stride(0), m, k, plan.topk, pw.data_ptr(), part.data_ptr(), 1, float(eps), plan.pair_row.data_ptr(),
                  plan.row_tile.data_ptr(), xq.data_ptr(), sf.data_ptr())
    launch(function("tcmoe", "moe_gather_quant"), ((m * (k // 32) + 255) // 256,), 256, 0, [mq])
    _KEEP.append((x, pw, part, plan))
    return xq, sf


# ------------------------------------------------------------------------------------------------ decode GEMVs
def tile_fp8(codes):
    """tile_fp8 (crates/model/src/formats.rs:96-118): e4m3 codes u8 [n][k] -> the mma.sync m16n8k16 A-fragment order the
    decode GEMV streams: per 64-row quad and 32-K step 2048 bytes = 4 row groups x 32 lanes x 16 bytes; lane (g = lane/4,
    t = lane%4) holds rows {g, g+8} x columns {2t, 2t+1, 8+2t, 9+2t, 16+2t, 17+2t, 24+2t, 25+2t}."""
    w = np.ascontiguousarray(codes, np.uint8)
    n, k = w.shape
    require(n % 64 == 0 and k % 32 == 0, "tile_fp8 needs n % 64 == 0 and k % 32 == 0")
    t = np.arange(4)[:, None]
    kk = np.concatenate([np.stack([2 * t[:, 0] + 8 * j, 2 * t[:, 0] + 8 * j + 1], axis=1) for j in range(4)], axis=1)   # [t][8]
    w6 = w.reshape(n // 64, 4, 2, 8, k // 32, 32)            # [q][rg][h][g][ks][c], row = rg*16 + h*8 + g
    a = w6[..., kk]                                          # [q][rg][h][g][ks][t][j]
    return np.ascontiguousarray(a.transpose(0, 4, 1, 3, 5, 2, 6)).reshape(-1)   # [q][ks][rg][g][t][h][j]


class RouteArgs(C.Structure):      # crates/engine/src/ops.rs:124-135
    _fields_ = [("scores", C.c_uint64), ("bias", C.c_uint64), ("ids", C.c_uint64), ("w", C.c_uint64), ("n_exp", C.c_int32), ("topk", C.c_int32),
                ("scale", C.c_float), ("nsum", C.c_int32)]


class RopeParams(C.Structure):     # crates/engine/src/ops.rs:42-61
    _fields_ = [("x", C.c_uint64), ("ldx", C.c_int32), ("n", C.c_int32), ("rows_per_token", C.c_int32), ("rope_off", C.c_int32),
                ("cos", C.c_uint64), ("sin", C.c_uint64), ("inverse", C.c_int32), ("quant", C.c_int32), ("ratio", C.c_int32), ("dst", C.c_uint64),
                ("pos_offset", C.c_int32), ("norm_w", C.c_uint64), ("norm_eps", C.c_float), ("dst_by_row", C.c_int32), ("q4", C.c_uint64),
                ("sf4", C.c_uint64)]


class GemvParams(C.Structure):     # crates/engine/src/ops.rs:63-115, mirror of cu/gemv.cu:19-71
    _fields_ = [("w", C.c_uint64), ("ws", C.c_uint64), ("x", C.c_uint64), ("out", C.c_uint64), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
                ("ldx", C.c_int32), ("ldo", C.c_int32), ("out_f32", C.c_int32), ("x_group_rows", C.c_int32), ("alpha", C.c_float),
                ("stage_steps", C.c_int32), ("plan", C.c_uint64), ("w_stride", C.c_uint64), ("mode", C.c_int32), ("swiglu_limit", C.c_float),
                ("prenorm_w", C.c_uint64), ("prenorm_eps", C.c_float), ("norm_part", C.c_uint64), ("norm_nslices", C.c_int32),
                ("ksplit_slots", C.c_int32), ("xq", C.c_uint64), ("xsq", C.c_uint64), ("oq", C.c_uint64), ("osq", C.c_uint64), ("sched", C.c_uint64),
                ("out2", C.c_uint64), ("ldo2", C.c_int32), ("n_split", C.c_int32), ("rope_cos", C.c_uint64), ("rope_sin", C.c_uint64),
                ("rope_pos", C.c_uint64), ("rope_head", C.c_int32), ("rope_off", C.c_int32), ("w_sh", C.c_uint64), ("route", RouteArgs),
                ("kvr", RopeParams), ("kvr_on", C.c_int32), ("_pad_kvr", C.c_int32), ("out_pos", C.c_uint64), ("iq_head", C.c_int32),
                ("iq_off", C.c_int32), ("sp", C.c_uint64), ("spart", C.c_uint64), ("sp_vloc", C.c_int32), ("sp_off", C.c_int32),
                ("xshift", C.c_int32), ("_padx", C.c_int32)]


class TvParams(C.Structure):       # crates/engine/src/ops.rs:1072-1103, mirror of cu/tcgemv.cu:10-31
    _fields_ = [("tmap", C.c_uint64), ("sfa", C.c_uint64), ("x", C.c_uint64), ("prenorm_w", C.c_uint64), ("norm_part", C.c_uint64), ("out", C.c_uint64),
                ("out2", C.c_uint64), ("rope_cos", C.c_uint64), ("rope_sin", C.c_uint64), ("meta", C.c_uint64), ("alpha", C.c_float), ("eps", C.c_float),
                ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("kpt", C.c_int32), ("ldx", C.c_int32), ("ldo", C.c_int32), ("ldo2", C.c_int32),
                ("n_split", C.c_int32), ("out_f32", C.c_int32), ("nslices", C.c_int32), ("rope_head", C.c_int32), ("rope_off", C.c_int32),
                ("partial", C.c_int32), ("group_rows", C.c_int32), ("kvr", RopeParams), ("kvr_on", C.c_int32), ("_pad2", C.c_int32)]


# the reference asserts these sizes (crates/engine/src/ops.rs:1165-1166)
assert C.sizeof(RopeParams) == 104 and C.sizeof(RouteArgs) == 48 and C.sizeof(GemvParams) == 432 and C.sizeof(TvParams) == 256

GEMV_STAGES = 4
SMEM_OPTIN = 227 * 1024            # ops::hw() for cc 10.0 (crates/engine/src/ops.rs:215)


def pick_ph(steps):                # crates/engine/src/ops.rs:290-292
    return 4 if steps >= 48 else 2 if steps >= 12 else 1


def gemv_smem(k, m, cs, tile_k=32, step_bytes=2048, prenorm=False):   # crates/engine/src/ops.rs:310-317
    mt = 8 if m <= 8 else 16
    ks = k // cs
    nsteps = ks // tile_k
    ss = min((nsteps + GEMV_STAGES - 1) // GEMV_STAGES, 12)
    return (GEMV_STAGES * ss * step_bytes + 2 * GEMV_STAGES * 8 + mt * (ks + 32) * 2 + mt * (ks // 32) * 4 + pick_ph(nsteps) * mt * 64 * 4
            + (ks * 2 if prenorm else 0) + ((mt * 64 + 4 * cs) * 4 if cs > 1 else 0))


def gemv_geometry(n, k, m, sms=148):
    """ops::gemv's choices for a dense FP8 weight (crates/engine/src/ops.rs:298-328, 331-474): K-split cluster size, pipeline
    depth, stage steps, grid, block and shared memory."""
    require(1 <= m <= 16, "gemv supports 1..=16 rows (ops.rs:342)")
    require(n % 64 == 0, "gemv needs n % 64 == 0 (ops.rs:343)")
    quads, unit = n // 64, 32
    cs = 1
    for c in (1, 2, 4, 8):                                    # pick_cluster (ops.rs:298-308)
        if k % (c * unit) == 0 and quads * c <= 2 * sms:
            cs = c
    while gemv_smem(k, m, cs) > SMEM_OPTIN and cs < 16 and k % (2 * cs * unit) == 0:   # gemv_cluster (ops.rs:319-328)
        cs *= 2
    ks = k // cs
    require(k % cs == 0 and ks % 32 == 0, f"bad split {cs} for k {k} (ops.rs:349)")
    require(ks // 32 <= 256, "the kernel stages at most 256 weight-scale bytes per scale row (cu/gemv.cu:194)")
    nsteps = ks // 32
    ss = min((nsteps + GEMV_STAGES - 1) // GEMV_STAGES, 12)
    smem = gemv_smem(k, m, cs)
    require(smem <= SMEM_OPTIN, f"gemv smem {smem} too large (ops.rs:354)")
    ph = pick_ph(nsteps)
    return {"nt": 1 if m <= 8 else 2, "ph": ph, "cs": cs, "ss": ss, "smem": smem, "grid": (quads, cs, 1), "block": (4 * ph + 1) * 32,
            "kernel": f"gemv_fp8_n{1 if m <= 8 else 2}_p{ph}"}


class GemvWeight:
    """Loader::fp8 (crates/engine/src/weights.rs:254-264): fragment-tiled codes + the raw 32x32 scale rows."""

    def __init__(self, codes, scales32):
        import torch
        codes = np.ascontiguousarray(codes, np.uint8)
        self.n, self.k = codes.shape
        self.w = torch.from_numpy(tile_fp8(codes)).cuda()
        self.s = torch.from_numpy(np.ascontiguousarray(scales32, np.uint8).reshape(self.n // 32, self.k // 32)).cuda()


def gemv_fp8(gw, x, out=None, alpha=1.0, pdl=False):
    """ops::gemv (crates/engine/src/ops.rs:331-474) for a dense FP8 weight with the Store epilogue: x bf16 [m][k] in (the
    kernel quantizes it 1x32 in shared memory, cu/quantblocks.cuh:7-57), bf16 [m][n] out."""
    import torch
    m, k = x.shape
    require(k == gw.k and x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0, "x bf16 [m][k]")
    geo = gemv_geometry(gw.n, gw.k, m, sm_count())
    if out is None:
        out = torch.empty(m, gw.n, dtype=torch.bfloat16, device=x.device)
    p = GemvParams()
    p.w, p.ws, p.x, p.out = gw.w.data_ptr(), gw.s.data_ptr(), x.data_ptr(), out.data_ptr()
    p.m, p.n, p.k, p.ldx, p.ldo = m, gw.n, gw.k, x.stride(0), out.stride(0)
    p.alpha, p.stage_steps = float(alpha), geo["ss"]
    f = function("gemv", geo["kernel"], geo["smem"], big_cluster=geo["cs"] > 8)
    launch(f, geo["grid"], geo["block"], geo["smem"], [p], cluster=(1, geo["cs"], 1), pdl=pdl)
    _KEEP.append((gw, x, out))
    return out


def tc_gemv_cluster(n, k, sms=148):   # crates/engine/src/ops.rs:1105-1107
    for c in (8, 5, 4, 2, 1):
        if k % (128 * c) == 0 and k // c <= 1024 and (n // 128) * c <= sms:
            return c if (n // 128) * c >= 96 else None
    return None


def tc_gemv_fp8(tw, x, out=None, alpha=1.0, pdl=False):
    """ops::tc_gemv (crates/engine/src/ops.rs:1118-1163): the tcgen05 decode GEMV, m <= 8; the whole K slice of a 128-row
    tile resident in shared memory, K split over a cluster with a push reduce."""
    import torch
    m, k = x.shape
    require(m <= 8 and tw.n % 128 == 0, "m <= 8 && n % 128 == 0 (ops.rs:1119)")
    require(k == tw.k and x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0, "x bf16 [m][k]")
    cs = tc_gemv_cluster(tw.n, tw.k, sm_count())
    require(cs is not None, f"tc_gemv: no split for n {tw.n} k {tw.k} (ops.rs:1120)")
    ks = k // cs
    kt = ks // 128
    smem = kt * (16384 + 1024 + 512 + 512) + 8 * ks * 2 + ks * 2 + 8 * 128 * 4 + 1040 * 4 + 1024
    require(smem <= SMEM_OPTIN, "tc_gemv shared memory")
    # the push reduce: every CTA expects (cs-1) * per * 4 bytes and sends per * 4 to each peer (cu/tcgemv.cu:62-74,196-208)
    per = ((m * 128 + cs - 1) // cs + 3) & ~3
    require(cs * per <= 1040, "receive buffer of the cluster reduce holds 1040 floats (ops.rs:1123)")
    if out is None:
        out = torch.empty(m, tw.n, dtype=torch.bfloat16, device=x.device)
    p = TvParams()
    p.tmap, p.sfa, p.x, p.out = tw.tmap128.data_ptr(), tw.sf.data_ptr(), x.data_ptr(), out.data_ptr()
    p.alpha, p.m, p.n, p.k, p.kpt, p.ldx, p.ldo = float(alpha), m, tw.n, tw.k, tw.k // 128, x.stride(0), out.stride(0)
    f = function("tcgemv", "tc_gemv_fp8", smem)
    launch(f, (tw.n // 128, cs, 1), 128, smem, [p], cluster=(1, cs, 1), pdl=pdl)
    _KEEP.append((tw, x, out))
    return out


# ------------------------------------------------------------------------------------------------ prefill expert GEMMs
class TmParams(C.Structure):       # crates/engine/src/ops.rs:1511-1534, mirror of cu/tcmoe.cu:137-160
    _fields_ = [("w", C.c_uint64), ("w_stride", C.c_uint64), ("k", C.c_int32), ("rt", C.c_int32), ("tb", C.c_uint64), ("sfb", C.c_uint64),
                ("tiles", C.c_uint64), ("ntiles", C.c_uint64), ("row_pair", C.c_uint64), ("row_w", C.c_uint64), ("aq", C.c_uint64),
                ("asf", C.c_uint64), ("ldaq", C.c_int32), ("akt", C.c_int32), ("limit", C.c_float), ("nq", C.c_int32), ("out", C.c_uint64),
                ("ldo", C.c_int32), ("flags", C.c_int32), ("sf_off", C.c_uint64)]


assert C.sizeof(TmParams) == 128
TM_SMEM = 4 * 16384 + 2 * (16 * 2080 + 4096) + 3 * 8 * 2176 + 40 * 512 + 2 * 32 * 33 * 4 + 1024   # crates/engine/src/ops.rs:1543
FP4_STEP = 2048 + 128                                                                             # crates/model/src/formats.rs:145


def tile_fp4(codes, scales):
    """tile_fp4 (crates/model/src/formats.rs:147-180): e2m1 codes u8 [n][k/2] (low nibble = even k) and UE8M0 scales u8
    [n][k/32] -> the image the mma.sync / prefill expert kernels stream: per 64-row quad and 64-K step 2048 bytes of
    codes (4 row groups x 32 lanes x 16 bytes; lane (g, t) holds, for j in 0..4, the bytes of rows {g, g+8} at K bytes
    {8j + t, 8j + 4 + t} of the step) followed by 128 bytes of scales (row group x g x {row g: 2 scales, row g+8: 2})."""
    w = np.ascontiguousarray(codes, np.uint8)
    s = np.ascontiguousarray(scales, np.uint8)
    n, kh = w.shape
    k = kh * 2
    require(n % 64 == 0 and k % 64 == 0 and s.shape == (n, k // 32), "tile_fp4 needs n % 64 == 0, k % 64 == 0, one scale per 32")
    steps = k // 64
    # byte column of a row = ks*32 + j*8 + half*4 + t;  row = q*64 + rg*16 + h*8 + g
    w8 = w.reshape(n // 64, 4, 2, 8, steps, 4, 2, 4)                        # [q][rg][h][g][ks][j][half][t]
    cw = np.ascontiguousarray(w8.transpose(0, 4, 1, 3, 7, 5, 2, 6))         # [q][ks][rg][g][t][j][h][half]
    s6 = s.reshape(n // 64, 4, 2, 8, steps, 2)                              # [q][rg][h][g][ks][c]
    cs = np.ascontiguousarray(s6.transpose(0, 4, 1, 3, 2, 5))               # [q][ks][rg][g][h][c]
    out = np.empty((n // 64, steps, FP4_STEP), np.uint8)
    out[:, :, :2048] = cw.reshape(n // 64, steps, 2048)
    out[:, :, 2048:] = cs.reshape(n // 64, steps, 128)
    return out.reshape(-1)


def interleave_gate_up(gate, up):
    """The row order of an expert's w13 image (crates/model/src/packing.rs:237-241): within each 64-row quad, rows 0-31 are
    gate rows 32q..32q+31 and rows 32-63 the matching up rows.  gate / up: [inter][...] -> [2*inter][...]."""
    inter = gate.shape[0]
    require(inter % 32 == 0 and up.shape == gate.shape, "inter % 32 == 0")
    g = gate.reshape(inter // 32, 32, -1)
    u = up.reshape(inter // 32, 32, -1)
    return np.ascontiguousarray(np.concatenate([g, u], axis=1)).reshape(2 * inter, -1)


def _maps8(base_tensor, cols, rows):
    """The eight activation tensor maps of PrefillMoe (crates/engine/src/model.rs:864-871): box rows 16, 32, ..., 128 over
    the same u8 [rows][cols] image, 128 bytes apart in one device allocation."""
    import torch
    require(base_tensor.data_ptr() % 16 == 0 and cols % 128 == 0, "activation image alignment")
    key = ("maps8", base_tensor.data_ptr(), cols, rows)
    if key in _TMAPS:
        return _TMAPS[key]
    host = np.zeros(8 * 128, np.uint8)
    for nb in range(1, 9):
        _check(lib().refk_tmap_u8_sw128(host[(nb - 1) * 128:].ctypes.data_as(C.c_void_p), base_tensor.data_ptr(), cols, rows, cols, 16 * nb))
    dev = torch.from_numpy(host).cuda()
    require(dev.data_ptr() % 64 == 0, "tensor maps must be 64-byte aligned in device memory")
    _TMAPS[key] = dev
    return dev


class MoeFp4Weights:
    """Per-expert tile_fp4 images of the gate/up (interleaved) and down projections of ``n_exp`` experts, as
    expert_shard_impl builds them for one tensor-parallel rank holding everything (packing.rs:209-254, tp = 1)."""

    def __init__(self, w13_codes, w13_scales, w2_codes, w2_scales):
        import torch
        e, n13, kh = w13_codes.shape
        self.n_exp, self.inter, self.dim = e, n13 // 2, kh * 2
        require(w2_codes.shape == (e, self.dim, self.inter // 2), "w2 codes [e][dim][inter/2]")
        require(self.dim % 128 == 0 and self.inter % 128 == 0, "this harness takes dim % 128 == 0 and inter % 128 == 0 (no K padding)")
        inter = self.inter
        img13 = [tile_fp4(interleave_gate_up(w13_codes[i, :inter], w13_codes[i, inter:]), interleave_gate_up(w13_scales[i, :inter], w13_scales[i, inter:]))
                 for i in range(e)]
        img2 = [tile_fp4(w2_codes[i], w2_scales[i]) for i in range(e)]
        self.w13 = torch.from_numpy(np.stack(img13)).cuda()
        self.w2 = torch.from_numpy(np.stack(img2)).cuda()
        self.w13_stride, self.w2_stride = self.w13.shape[1], self.w2.shape[1]


def tc_moe(weights, plan, xq, sf, swiglu_limit=0.0, out=None):
    """tc_moe_w13 then tc_moe_w2 as Rank::ffn_prefill launches them (crates/engine/src/model.rs:3125-3166, the path without
    the row-major expert image): grid = SM count, 512 threads, TM_SMEM bytes.  xq / sf: moe_gather_quant's outputs.
    Returns (aq u8 [rows + 128][ldaq] in kpos32 order, asf atoms, ypair f32 [pairs][dim]); ``out``: the same three buffers
    from an earlier call, reused (timing loops)."""
    import torch
    dim, inter = weights.dim, weights.inter
    rows, slack = plan.p, plan.p + 128
    require(xq.shape == (slack, dim) and xq.dtype == torch.uint8, "xq is moe_gather_quant's [rows + 128][dim] image")
    # the kernel keeps the activation scale atoms of all K tiles of a token tile in 40 slots (cu/tcmoe.cu:171)
    require(dim // 128 <= 40 and inter // 128 <= 40, "K <= 5120 (SFB_MAX = 40 scale atoms per token tile)")
    require((2 * inter) % 64 == 0 and inter % 64 == 0, "model.rs:854: (2 * inter) % 64 == 0 && kpad % 64 == 0")
    ntile_cap = rows // 128 + plan.n_exp
    require(ntile_cap <= 1024, "tile list (TM_MAX_TILES)")
    ldaq, akt = inter, inter // 128                       # kpad = inter: model.rs:860-861
    dev = xq.device
    if out is not None:
        aq, asf, ypair = out
        require(aq.shape == (slack, ldaq) and asf.numel() == ntile_cap * akt * 512 and ypair.shape == (rows, dim), "reused output buffers")
    else:
        aq = torch.zeros(slack, ldaq, dtype=torch.uint8, device=dev)
        asf = torch.zeros(ntile_cap * akt * 512, dtype=torch.uint8, device=dev)
        ypair = torch.zeros(rows, dim, dtype=torch.float32, device=dev)
    tb13, tb2 = _maps8(xq, dim, slack), _maps8(aq, ldaq, slack)
    sms = sm_count()
    p13 = TmParams(weights.w13.data_ptr(), weights.w13_stride, dim, (2 * inter + 127) // 128, tb13.data_ptr(), sf.data_ptr(), plan.tiles.data_ptr(),
                   plan.ntiles.data_ptr(), plan.row_pair.data_ptr(), plan.row_w.data_ptr(), aq.data_ptr(), asf.data_ptr(), ldaq, akt,
                   float(swiglu_limit), 2 * inter // 64, 0, 0, 0, 0)
    p2 = TmParams(weights.w2.data_ptr(), weights.w2_stride, inter, dim // 128, tb2.data_ptr(), asf.data_ptr(), plan.tiles.data_ptr(),
                  plan.ntiles.data_ptr(), plan.row_pair.data_ptr(), plan.row_w.data_ptr(), aq.data_ptr(), asf.data_ptr(), ldaq, akt,
                  float(swiglu_limit), dim // 64, ypair.data_ptr(), dim, 0, 0)
    launch(function("tcmoe", "tc_moe_w13", smem=TM_SMEM), (sms,), 512, TM_SMEM, [p13])
    launch(function("tcmoe", "tc_moe_w2", smem=TM_SMEM), (sms,), 512, TM_SMEM, [p2])
    _KEEP.append((weights, plan, xq, sf, tb13, tb2))
    return aq, asf, ypair


def unpermute_k32(codes_rows):
    """Inverse of the kpos32 order inside every 32-K block: u8 [rows][k] as moe_gather_quant / tc_moe_w13 store them ->
    natural K order."""
    a = np.asarray(codes_rows, np.uint8)
    rows, k = a.shape
    pos = np.array([kpos32(j) for j in range(32)])
    return np.ascontiguousarray(a.reshape(rows, k // 32, 32)[:, :, pos]).reshape(rows, k)
