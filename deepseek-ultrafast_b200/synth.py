"""Synthetic (random-init) weights of the benchmark shapes, generated and packed on the GPU with torch ops.

Checkpoints cannot be downloaded in this environment, so benchmarks and full-size parity tests draw weights
~N(0, std), quantize them (FP8 128x128 / 32x32, MXFP4 1x32) and lay them out as the library's 128x128 tile
records -- all on the device, because 256 experts of 4096x7168 + 7168x2048 are too slow to build on the host.
This is input generation, not the hot path.  ``unpack_*`` turn tile records back into plain codes/scales on the
host so the CPU oracle can be fed exactly what the kernels read.
"""
import numpy as np

REC_FP4 = 8192 + 512
REC_FP8_MX = 16384 + 512
REC_FP8_DS = 16384


def _atoms(torch, sc):
    """sc u8 [rt*128][kt*4] -> [rt][kt][512] in the tcgen05 scale-factor atom order."""
    n, kb = sc.shape
    rt, kt = n // 128, kb // 4
    a = sc.view(rt, 4, 32, kt, 4).permute(0, 3, 2, 1, 4)  # [rt][kt][r%32][r/32][b]
    return a.reshape(rt, kt, 512)


def fp4_expert_tiles(torch, n, k, std, gen, gate_up, device):
    """One expert matrix [n][k] ~ N(0,std) -> u8 tile records [n/128 * k/128 * 8704]."""
    w = torch.randn(n, k, generator=gen, device=device, dtype=torch.float32) * std
    w = w.bfloat16().float()
    wb = w.view(n, k // 32, 32)
    amax = wb.abs().amax(-1).clamp_min(6.0 * 1.1754944e-38)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-126, 127)
    # guard against log2 rounding: scale must be >= amax/6
    e = torch.where(torch.exp2(e) * 6.0 < amax, e + 1, e)
    sc = (e + 127).to(torch.uint8)
    v = wb / torch.exp2(e).unsqueeze(-1)
    mag = v.abs().clamp_max(6.0)
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=device)
    code = torch.bucketize(mag, bounds).to(torch.uint8) | ((v < 0).to(torch.uint8) << 3)
    code = code.view(n, k)
    codes = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()  # [n][k/2]
    if gate_up:
        inter = n // 2
        pr = torch.arange(n, device=device)
        src = torch.where((pr % 16) // 8 == 1, inter, 0) + (pr // 16) * 8 + pr % 8
        codes, sc = codes[src], sc[src]
    rt, kt = n // 128, k // 128
    ct = codes.view(rt, 128, kt, 64).permute(0, 2, 1, 3).reshape(rt, kt, 8192)
    return torch.cat([ct, _atoms(torch, sc.contiguous())], dim=2).reshape(-1)


def fp4_experts(torch, n_experts, n, k, std, seed, gate_up, device, first_expert=0):
    """Experts first_expert .. first_expert + n_experts - 1 of the stream named by `seed`: every expert is drawn from its
    own generator state (seed, global expert id), so an expert-parallel shard holds exactly the experts the unsharded
    weight holds at those ids."""
    gen = torch.Generator(device=device)
    per = (n // 128) * (k // 128) * REC_FP4
    out = torch.empty(n_experts * per, dtype=torch.uint8, device=device)
    for e in range(n_experts):
        gen.manual_seed(seed * 1000003 + first_expert + e)
        out[e * per:(e + 1) * per] = fp4_expert_tiles(torch, n, k, std, gen, gate_up, device)
    return out


def fp8_dense(torch, mode_mx, n, k, std, seed, device, k_slice=None, n_slice=None):
    """Dense weight [n][k] ~ N(0,std) -> (tile records u8, ds scales f32 [n/128][k/128] or None).
    ``k_slice`` = (k0, k1), multiples of 128: only columns k0..k1 of the same [n][k] weight are quantized and packed (the
    K-shard of a tensor-parallel rank; block scales do not straddle a multiple of 128, so the shard's codes and scales
    are those of the whole weight); ``n_slice`` = (n0, n1) likewise selects rows."""
    gen = torch.Generator(device=device).manual_seed(seed)
    w = (torch.randn(n, k, generator=gen, device=device, dtype=torch.float32) * std).bfloat16().float()
    if k_slice is not None:
        w = w[:, k_slice[0]:k_slice[1]].contiguous()
        k = k_slice[1] - k_slice[0]
    if n_slice is not None:      # rows n0..n1 (multiples of 128): the shard of a rank that owns those OUTPUT columns
        w = w[n_slice[0]:n_slice[1]].contiguous()
        n = n_slice[1] - n_slice[0]
    rt, kt = n // 128, k // 128
    if mode_mx:
        wb = w.view(n // 32, 32, k // 32, 32)
        amax = wb.abs().amax(dim=(1, 3)).clamp_min(1e-30)
        e = torch.ceil(torch.log2(amax / 448.0)).clamp(-126, 127)
        e = torch.where(torch.exp2(e) * 448.0 < amax, e + 1, e)
        q = (wb / torch.exp2(e)[:, None, :, None]).to(torch.float8_e4m3fn).view(torch.uint8).view(n, k)
        sc_rows = (e + 127).to(torch.uint8).repeat_interleave(32, dim=0)  # per row, per 32-K
        ct = q.view(rt, 128, kt, 128).permute(0, 2, 1, 3).reshape(rt, kt, 16384)
        return torch.cat([ct, _atoms(torch, sc_rows.contiguous())], dim=2).reshape(-1), None
    wb = w.view(rt, 128, kt, 128)
    amax = wb.abs().amax(dim=(1, 3))
    sc = torch.where(amax == 0, torch.ones_like(amax), amax / 448.0)
    q = (wb / sc[:, None, :, None]).to(torch.float8_e4m3fn).view(torch.uint8)
    return q.permute(0, 2, 1, 3).reshape(-1).contiguous(), sc.contiguous()


# ---- host-side inverses (numpy) ----
def unpack_fp4(tiles, n, k, gate_up):
    """tile records (numpy u8) -> codes [n][k/2], scales [n][k/32] in the caller's row order (gate rows, then up)."""
    rt, kt = n // 128, k // 128
    t = np.asarray(tiles).reshape(rt, kt, REC_FP4)
    codes = t[:, :, :8192].reshape(rt, kt, 128, 64).transpose(0, 2, 1, 3).reshape(n, k // 2)
    at = t[:, :, 8192:].reshape(rt, kt, 32, 4, 4).transpose(0, 3, 2, 1, 4)  # [rt][r/32][r%32][kt][b]
    sc = at.reshape(n, k // 32)
    if gate_up:
        inter = n // 2
        pr = np.arange(n)
        src = np.where((pr % 16) // 8 == 1, inter, 0) + (pr // 16) * 8 + pr % 8
        c2, s2 = np.empty_like(codes), np.empty_like(sc)
        c2[src], s2[src] = codes, sc
        codes, sc = c2, s2
    return np.ascontiguousarray(codes), np.ascontiguousarray(sc)


def unpack_fp8(tiles, mode_mx, n, k):
    rt, kt = n // 128, k // 128
    rec = REC_FP8_MX if mode_mx else REC_FP8_DS
    t = np.asarray(tiles).reshape(rt, kt, rec)
    codes = t[:, :, :16384].reshape(rt, kt, 128, 128).transpose(0, 2, 1, 3).reshape(n, k)
    if not mode_mx:
        return np.ascontiguousarray(codes), None
    at = t[:, :, 16384:].reshape(rt, kt, 32, 4, 4).transpose(0, 3, 2, 1, 4).reshape(n, k // 32)
    return np.ascontiguousarray(codes), np.ascontiguousarray(at[::32])
