"""Checkpoint-facing loaders: the safetensors reader and the mapping of on-disk FP8 / FP4 tensors to tile records
(csrc/loader.cc), against files written here byte by byte in the safetensors layout (8-byte little-endian header length,
JSON header, raw tensor data) and against the library's own packers on the same arrays."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import oracle


def write_safetensors(path, tensors, metadata=None):
    """tensors: name -> (dtype string, shape, bytes-like)."""
    hdr, blobs, off = {}, [], 0
    if metadata:
        hdr["__metadata__"] = metadata
    for name, (dt, shape, data) in tensors.items():
        b = bytes(data)
        hdr[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(hdr).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def _dense(seed, n, k):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().view(torch.uint16).numpy()
    return oracle.quant_fp8_weight(oracle.MODE_MX, w)


def _experts(seed, e, inter, dim):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(e):
        w1 = (torch.randn(inter, dim, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
        w3 = (torch.randn(inter, dim, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
        w2 = (torch.randn(dim, inter, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
        out.append([oracle.quant_fp4_weight(x) for x in (w1, w3, w2)])
    return out


@pytest.fixture
def ckpt_dir(tmp_path):
    wq, ws = _dense(1, 256, 384)
    ex = _experts(2, 3, 128, 256)
    a = {"layers.0.attn.wq_b.weight": ("F8_E4M3", wq.shape, wq.tobytes()), "layers.0.attn.wq_b.scale": ("F8_E8M0", ws.shape, ws.tobytes()),
         "layers.0.norm.weight": ("BF16", (384,), np.arange(384, dtype=np.uint16).tobytes())}
    b = {}
    for e, ((c1, s1), (c3, s3), (c2, s2)) in enumerate(ex):
        for nm, c, s in (("w1", c1, s1), ("w3", c3, s3), ("w2", c2, s2)):
            b[f"layers.0.ffn.experts.{e}.{nm}.weight"] = ("I8", c.shape, c.tobytes())
            b[f"layers.0.ffn.experts.{e}.{nm}.scale"] = ("F8_E8M0", s.shape, s.tobytes())
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", a, metadata={"format": "pt", "note": 'a "quoted" value, [brackets] {braces}'})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", b)
    (tmp_path / "tokenizer.json").write_text("{}")
    return tmp_path, (wq, ws), ex


def test_reader_indexes_every_shard_and_returns_the_bytes(pkg, ckpt_dir):
    d, (wq, ws), ex = ckpt_dir
    ck = pkg.Checkpoint(str(d))
    try:
        assert len(ck) == 3 + 3 * 6
        dt, shape, raw = ck.tensor("layers.0.attn.wq_b.weight")
        assert dt == "F8_E4M3" and shape == wq.shape and (raw.reshape(shape) == wq).all()
        dt, shape, raw = ck.tensor("layers.0.norm.weight")
        assert dt == "BF16" and shape == (384,) and (raw.view(np.uint16) == np.arange(384)).all()
        dt, shape, raw = ck.tensor("layers.0.ffn.experts.2.w2.scale")
        assert shape == ex[2][2][1].shape and (raw.reshape(shape) == ex[2][2][1]).all()
        with pytest.raises(pkg.DsufError, match="not in checkpoint"):
            ck.tensor("layers.9.nothing")
    finally:
        ck.close()
    one = pkg.Checkpoint(str(d / "model-00001-of-00002.safetensors"))   # a single file works as well
    assert len(one) == 3
    one.close()


def test_fp8_dense_loader_equals_the_packer_on_the_same_arrays(pkg, ckpt_dir):
    d, (wq, ws), _ = ckpt_dir
    ck = pkg.Checkpoint(str(d))
    try:
        tiles, n, k = ck.fp8_dense_tiles("layers.0.attn.wq_b")
        assert (n, k) == wq.shape and (tiles == pkg.pack_fp8_weight(pkg.MODE_MX, wq, ws)).all()
        # a row shard (what a rank that owns output columns 128..255 loads): the records of those rows alone
        part, n2, _ = ck.fp8_dense_tiles("layers.0.attn.wq_b", rows=(128, 256))
        assert n2 == 128 and (part == pkg.pack_fp8_weight(pkg.MODE_MX, wq[128:], ws[4:])).all()
        with pytest.raises(pkg.DsufError, match="multiples of 32"):
            ck.fp8_dense_tiles("layers.0.attn.wq_b", rows=(16, 256))
        with pytest.raises(pkg.DsufError, match="not in checkpoint"):
            ck.fp8_dense_tiles("layers.0.attn.wkv")
    finally:
        ck.close()


def test_expert_loader_equals_the_packer_with_gate_up_interleave(pkg, ckpt_dir):
    d, _, ex = ckpt_dir
    ck = pkg.Checkpoint(str(d))
    try:
        o13, o2 = ck.fp4_expert_tiles("layers.0", 1, 3, 256, 128)    # an expert-parallel rank's range
        per13, per2 = o13.size // 2, o2.size // 2
        for i, e in enumerate((1, 2)):
            (c1, s1), (c3, s3), (c2, s2) = ex[e]
            want13 = pkg.pack_fp4_weight(np.concatenate([c1, c3]), np.concatenate([s1, s3]), True)
            assert (o13[i * per13:(i + 1) * per13] == want13).all()
            assert (o2[i * per2:(i + 1) * per2] == pkg.pack_fp4_weight(c2, s2, False)).all()
        with pytest.raises(pkg.DsufError, match="experts.3"):
            ck.fp4_expert_tiles("layers.0", 2, 4, 256, 128)           # expert 3 does not exist
        with pytest.raises(pkg.DsufError, match="shape"):
            ck.fp4_expert_tiles("layers.0", 0, 1, 256, 256)           # wrong intermediate size
    finally:
        ck.close()


def test_malformed_files_are_rejected_with_a_message(pkg, tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")                 # header length beyond the file
    with pytest.raises(pkg.DsufError, match="header length"):
        pkg.Checkpoint(str(p))
    p.write_bytes(struct.pack("<Q", 9) + b'{"a": [1}')               # not the safetensors header grammar
    with pytest.raises(pkg.DsufError, match="malformed"):
        pkg.Checkpoint(str(p))
    h = json.dumps({"t": {"dtype": "U8", "shape": [4], "data_offsets": [0, 400]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"abcd")           # data range beyond the file
    with pytest.raises(pkg.DsufError, match="malformed"):
        pkg.Checkpoint(str(p))
    with pytest.raises(pkg.DsufError, match="no such file"):
        pkg.Checkpoint(str(tmp_path / "absent"))
    (tmp_path / "empty").mkdir()
    with pytest.raises(pkg.DsufError, match="no \\*.safetensors"):
        pkg.Checkpoint(str(tmp_path / "empty"))


@pytest.mark.gpu
def test_loaded_weights_run_like_weights_packed_from_arrays(pkg, ctx, ckpt_dir):
    """End to end on the GPU: a dense FP8 weight and three experts read from the checkpoint files give the outputs of the
    same weights handed over as arrays."""
    d, (wq, ws), ex = ckpt_dir
    ck = pkg.Checkpoint(str(d))
    try:
        g = torch.Generator().manual_seed(5)
        x = torch.randn(5, 384, generator=g).bfloat16().cuda()
        a = pkg.gemv(ctx, ck.load_fp8_dense(ctx, "layers.0.attn.wq_b"), x)
        b = pkg.gemv(ctx, pkg.Weight.dense_fp8(ctx, pkg.MODE_MX, wq, ws), x)
        torch.cuda.synchronize()
        assert torch.equal(a.view(torch.uint16), b.view(torch.uint16))
        W13, W2 = ck.load_experts(ctx, "layers.0", 0, 3, 256, 128)
        c13 = np.stack([np.concatenate([e[0][0], e[1][0]]) for e in ex]); s13 = np.stack([np.concatenate([e[0][1], e[1][1]]) for e in ex])
        c2 = np.stack([e[2][0] for e in ex]); s2 = np.stack([e[2][1] for e in ex])
        V13, V2 = pkg.Weight.experts_fp4(ctx, c13, s13, True), pkg.Weight.experts_fp4(ctx, c2, s2, False)
        T, K = 16, 2
        xm = torch.randn(T, 256, generator=g).bfloat16().cuda()
        logits = torch.randn(T, 3, generator=g).cuda()
        outs = []
        for w13, w2 in ((W13, W2), (V13, V2)):
            layer = pkg.MoeLayer(ctx, w13, w2, T, K, pkg.MODE_MX)
            ids = torch.empty(T, K, dtype=torch.int32, device="cuda"); w = torch.empty(T, K, dtype=torch.float32, device="cuda")
            y = torch.empty(T, 256, dtype=torch.bfloat16, device="cuda")
            layer.forward(xm, ids, w, y, route=(pkg.SCORE_SOFTMAX, logits, None, 1.0))
            torch.cuda.synchronize()
            outs.append(y.clone())
        assert ctx.status().code == 0 and torch.equal(outs[0].view(torch.uint16), outs[1].view(torch.uint16))
    finally:
        ck.close()
