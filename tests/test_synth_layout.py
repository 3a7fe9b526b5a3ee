"""The torch-side synthetic-weight generator (used at full benchmark sizes) produces exactly the tile-record layout of
the library's own packers; checked on CPU tensors."""
import numpy as np
import torch

import oracle


def _synth(pkg):
    import importlib
    return importlib.import_module(pkg.__name__ + ".synth")


def test_fp4_generator_layout_matches_packer(pkg):
    synth = _synth(pkg)
    n, k = 256, 256
    for gate_up in (False, True):
        gen = torch.Generator().manual_seed(3)
        tiles = synth.fp4_expert_tiles(torch, n, k, 0.02, gen, gate_up, "cpu").numpy()
        codes, sc = synth.unpack_fp4(tiles, n, k, gate_up)
        assert (pkg.pack_fp4_weight(codes, sc, gate_up) == tiles).all()
        # scales are the smallest power of two with amax/scale <= 6 and the codes decode near the weights
        deq = oracle.dequant_fp4(codes, sc)
        gen = torch.Generator().manual_seed(3)
        w = (torch.randn(n, k, generator=gen) * 0.02).bfloat16().float().numpy()
        assert np.abs(deq - w).max() <= np.abs(w).max() * 0.26
        co, so = oracle.quant_fp4_weight(oracle.f32_to_bf16(w))
        assert (so == sc).all()
        assert (co != codes).mean() < 0.02   # only exact rounding ties may differ


def test_fp8_generator_layout_matches_packer(pkg):
    synth = _synth(pkg)
    n, k = 256, 384
    for mx in (True, False):
        tiles, sds = synth.fp8_dense(torch, mx, n, k, 0.02, 5, "cpu")
        codes, sc = synth.unpack_fp8(tiles.numpy(), mx, n, k)
        mode = pkg.MODE_MX if mx else pkg.MODE_DS
        assert (pkg.pack_fp8_weight(mode, codes, sc) == tiles.numpy()).all()
        gen = torch.Generator().manual_seed(5)
        w = (torch.randn(n, k, generator=gen) * 0.02).bfloat16()
        qo, so = oracle.quant_fp8_weight(mode, w.view(torch.uint16).numpy())
        got_s = sc if mx else sds.numpy()
        assert (so == got_s).all()
        assert (qo != codes).mean() < 1e-3


def test_shards_are_slices_of_one_weight_set(pkg):
    """Expert-parallel shards (experts by global id) and tensor-parallel shards (a K slice of the dense weight) hold the
    bytes of the unsharded weights, so a W-rank stack computes the same function as the single-GPU one."""
    synth = _synth(pkg)
    n, k, e = 128, 256, 6
    whole = synth.fp4_experts(torch, e, n, k, 0.02, 9, False, "cpu")
    per = whole.numel() // e
    for lo, cnt in ((0, 3), (3, 3), (4, 2)):
        part = synth.fp4_experts(torch, cnt, n, k, 0.02, 9, False, "cpu", first_expert=lo)
        assert (part == whole[lo * per:(lo + cnt) * per]).all()
    n, k = 256, 512
    for mx in (True, False):
        mode = pkg.MODE_MX if mx else pkg.MODE_DS
        tiles, sds = synth.fp8_dense(torch, mx, n, k, 0.02, 4, "cpu")
        codes, sc = synth.unpack_fp8(tiles.numpy(), mx, n, k)
        for k0, k1 in ((0, 256), (256, 512), (128, 256)):
            pt, ps = synth.fp8_dense(torch, mx, n, k, 0.02, 4, "cpu", k_slice=(k0, k1))
            pc, psc = synth.unpack_fp8(pt.numpy(), mx, n, k1 - k0)
            assert (pc == codes[:, k0:k1]).all()
            if mx:
                assert (psc == sc[:, k0 // 32:k1 // 32]).all()
            else:
                assert (ps.numpy() == sds.numpy()[:, k0 // 128:k1 // 128]).all()
