"""CPU oracle tests: the pure-PyTorch op implementations against torch.nn.functional / autograd."""
import math

import pytest
import torch
import torch.nn.functional as F

from chronicals_b200 import ops
from chronicals_b200.ops import ref


def test_rmsnorm_matches_formula():
    x, w = torch.randn(5, 64), torch.rand(64) + 0.5
    y = ops.rmsnorm(x, w, 1e-6)
    want = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert torch.allclose(y, want, atol=1e-6)
    y2, h = ops.add_rmsnorm(x, 2 * x, w)
    assert torch.allclose(h, 3 * x) and torch.allclose(y2, ops.rmsnorm(3 * x, w), atol=1e-6)


def test_glu_variants():
    gu = torch.randn(7, 32, dtype=torch.float64)
    g, u = gu.chunk(2, -1)
    assert torch.allclose(ops.swiglu(gu), F.silu(g) * u)
    assert torch.allclose(ops.geglu(gu), F.gelu(g, approximate="tanh") * u)


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_is_a_rotation_and_matches_hf(interleaved):
    T, H, D = 12, 3, 16
    x = torch.randn(T, H, D, dtype=torch.float64)
    cos, sin = ref.rope_cache(64, D, 1e4)
    pos = torch.tensor([0, 1, 2, 3, 0, 1, 2, 0, 1, 2, 3, 4])
    y = ref.apply_rope(x, cos, sin, pos, interleaved)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    back = ref.apply_rope(y, cos, sin, pos, interleaved, inverse=True)
    assert torch.allclose(back, x, atol=1e-5)
    if not interleaved:      # HF rotate_half convention
        c = torch.cat((cos[pos], cos[pos]), -1)[:, None].double()
        s = torch.cat((sin[pos], sin[pos]), -1)[:, None].double()
        rot = torch.cat((-x[..., D // 2:], x[..., : D // 2]), -1)
        assert torch.allclose(y, x * c + rot * s, atol=1e-5)


def test_rope_scaling_variants_are_finite_and_ordered():
    base, _ = ref.rope_inv_freq(64, 1e4)
    for sc in ({"type": "linear", "factor": 2.0}, {"type": "ntk", "factor": 4.0},
               {"type": "yarn", "factor": 4.0, "original_max_position_embeddings": 2048},
               {"type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                "original_max_position_embeddings": 8192}):
        inv, scale = ref.rope_inv_freq(64, 1e4, sc)
        assert torch.isfinite(inv).all() and (inv <= base * 1.0001).all() and scale >= 1.0


def test_qk_rope_packed_buffer_cpu():
    T, hq, hk, d = 9, 4, 2, 8
    qkv = torch.randn(T, (hq + 2 * hk) * d)
    cos, sin = ref.rope_cache(32, d, 1e6)
    pos = torch.arange(T) % 5
    out = ops.qk_rope_(qkv, cos, sin, pos, hq, hk, d)
    q = ref.apply_rope(qkv[:, :hq * d].reshape(T, hq, d), cos, sin, pos)
    assert torch.allclose(out[:, :hq * d], q.reshape(T, -1), atol=1e-6)
    assert torch.equal(out[:, (hq + hk) * d:], qkv[:, (hq + hk) * d:])


def test_attention_varlen_matches_masked_sdpa():
    T, hq, hk, d = 40, 4, 2, 16
    q, k, v = torch.randn(T, hq, d), torch.randn(T, hk, d), torch.randn(T, hk, d)
    cu = torch.tensor([0, 10, 11, 33], dtype=torch.int32)
    o = ops.attention_varlen(q, k, v, cu, 22)
    doc = torch.full((T,), -1)
    for i, (a, b) in enumerate(zip(cu[:-1].tolist(), cu[1:].tolist())):
        doc[a:b] = i
    mask = (doc[:, None] == doc[None, :]) & torch.ones(T, T, dtype=torch.bool).tril() & (doc[:, None] >= 0)
    mask |= torch.eye(T, dtype=torch.bool)
    want = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1).repeat_interleave(2, 0)[None],
                                          v.transpose(0, 1).repeat_interleave(2, 0)[None], attn_mask=mask)[0].transpose(0, 1)
    assert torch.allclose(o[:33], want[:33], atol=1e-5)
    assert o[33:].abs().max() == 0


@pytest.mark.parametrize("smoothing,z", [(0.0, 0.0), (0.1, 0.0), (0.0, 1e-3), (0.05, 1e-4)])
@pytest.mark.parametrize("bias", [False, True])
def test_chunked_linear_ce_matches_dense_with_grads(smoothing, z, bias):
    torch.manual_seed(0)
    T, H, V = 33, 24, 101
    h = torch.randn(T, H, dtype=torch.float64, requires_grad=True)
    w = torch.randn(V, H, dtype=torch.float64, requires_grad=True)
    b = torch.randn(V, dtype=torch.float64, requires_grad=True) if bias else None
    y = torch.randint(0, V, (T,))
    y[::5] = -100
    dense = ref.linear_cross_entropy_dense(h, w, y, b, -100, smoothing, z)
    gd = torch.autograd.grad(dense, [h, w] + ([b] if bias else []))
    ch = ref.linear_cross_entropy_chunked(h, w, y, b, -100, smoothing, z, "mean", chunk_size=16)
    gc = torch.autograd.grad(ch, [h, w] + ([b] if bias else []))
    assert abs(dense.item() - ch.item()) < 1e-4
    for a, c in zip(gd, gc):
        assert torch.allclose(a.float(), c.float(), atol=1e-5), (a - c).abs().max()
    # equals torch's own cross entropy when no z-loss
    if z == 0:
        lg = (h @ w.t() + (b if bias else 0)).float()
        assert abs(F.cross_entropy(lg, y, ignore_index=-100, label_smoothing=smoothing).item() - ch.item()) < 1e-4


def test_linear_ce_all_ignored_is_zero_not_nan():
    h, w = torch.randn(4, 8, requires_grad=True), torch.randn(16, 8, requires_grad=True)
    loss = ops.linear_cross_entropy(h, w, torch.full((4,), -100))
    loss.backward()
    assert loss.item() == 0 and torch.isfinite(h.grad).all()


def test_adamw_reference_step_matches_torch():
    torch.manual_seed(0)
    p = torch.randn(50)
    q = torch.nn.Parameter(p.clone())
    m, v = torch.zeros(50), torch.zeros(50)
    opt = torch.optim.AdamW([q], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for t in range(1, 4):
        g = torch.randn(50)
        q.grad = g.clone()
        opt.step()
        ref.adamw_step_(p, g, m, v, t, 1e-2, 0.9, 0.95, 1e-8, 0.1)
    assert torch.allclose(p, q.detach(), atol=1e-6)


def test_mxfp8_quantization_is_exact_power_of_two_scaling():
    torch.manual_seed(0)
    x = torch.randn(4, 64) * torch.tensor([1e-3, 1.0, 300.0, 5e4])[:, None]
    q, s = ref.mxfp8_quantize(x)
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.uint8 and s.shape == (4, 2)
    scale = torch.exp2(s.float() - 127)
    amax = x.reshape(4, 2, 32).abs().amax(-1)
    assert (amax / scale <= 448.0 + 1e-3).all() and (amax / scale > 224.0 - 1e-3).all()
    back = ref.mxfp8_dequantize(q, s)
    assert ((back - x).abs() <= 0.0625 * amax.repeat_interleave(32, -1).reshape(4, 64) + 1e-12).all()
    zq, zs = ref.mxfp8_quantize(torch.zeros(1, 32))
    assert zq.float().abs().max() == 0


def test_mx_scale_atoms_layout_and_block_scaled_product_oracle():
    """The packed scale layout of the block-scaled tensor-core GEMM (512-byte atoms of 128 rows x 4 blocks,
    byte (r % 32) * 16 + (r // 32 % 4) * 4 + kb % 4) round-trips, pads with scale 1.0, and the CPU path of
    the block-scaled product equals the dequantise-then-multiply oracle."""
    from chronicals_b200.utils import fp8_utils as F8
    s = torch.randint(100, 140, (200, 5), dtype=torch.uint8)
    p = F8.pack_mx_scales(s)
    assert p.numel() == 2 * 2 * 512
    assert torch.equal(F8.unpack_mx_scales(p, 200, 5), s)
    for r, kb in [(0, 0), (33, 1), (130, 4), (199, 3)]:
        idx = ((r // 128) * 2 + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4
        assert p[idx] == s[r, kb]
    written = torch.zeros(p.numel(), dtype=torch.bool)
    for r in range(200):
        for kb in range(5):
            written[((r // 128) * 2 + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4] = True
    assert (p[~written] == 127).all()
    x, w = torch.randn(200, 160), torch.randn(136, 160)
    aq, sa = F8.mxfp8_quantize_packed(x)
    bq, sb = F8.mxfp8_quantize_packed(w)
    y = F8.mxfp8_block_scaled_matmul(aq, sa, bq, sb)
    assert torch.equal(y, ref.mxfp8_linear(x, w))
    # tiles of 192 rows (the CTA-pair kernel's B operand): each tile padded to 256 rows = two atoms per 4 blocks
    s2 = torch.randint(100, 140, (400, 5), dtype=torch.uint8)
    p2 = F8.pack_mx_scales(s2, 192)
    assert p2.numel() == 3 * 2 * 2 * 512 and torch.equal(F8.unpack_mx_scales(p2, 400, 5, 192), s2)
    for r, kb in [(0, 0), (130, 1), (191, 4), (192, 0), (399, 3)]:
        t, rr = divmod(r, 192)
        atom = (2 * t + rr // 128) * 2 + kb // 4
        assert p2[atom * 512 + (rr % 32) * 16 + ((rr // 32) % 4) * 4 + kb % 4] == s2[r, kb]
    bq, sb = F8.mxfp8_quantize_packed(w, tile_rows=192)
    assert torch.equal(F8.mxfp8_block_scaled_matmul(aq, sa, bq, sb, b_tile_rows=192), ref.mxfp8_linear(x, w))


def test_wgrad_cpu_path_matches_matmul():
    from chronicals_b200 import ops
    dy, x = torch.randn(64, 24), torch.randn(64, 40)
    assert torch.allclose(ops.wgrad(dy, x), dy.t() @ x, atol=1e-5)


def test_blockwise_8bit_roundtrip():
    x = torch.randn(1000)
    q, a = ref.quantize_blockwise_8bit(x)
    back = ref.dequantize_blockwise_8bit(q, a, x.shape)
    assert (back - x).abs().max() <= a.max() / 127 * 0.51 + 1e-6


def test_clip_coef():
    c = ref.clip_coef_from_sqnorm(torch.tensor(16.0), 1.0)
    assert abs(c.item() - 1.0 / (4.0 + 1e-6)) < 1e-6
    assert ref.clip_coef_from_sqnorm(torch.tensor(0.01), 1.0).item() == 1.0


def test_fma_pipe_exp2_constants_and_bit_arithmetic():
    """The softmax kernels compute part of their exponentials without the special-function unit (``ex2_fma`` in
    ``csrc/common.cuh``): x = n + f, a cubic for 2^f, n added to the exponent field.  The same arithmetic in numpy
    float32, with the constants read from the source, stays within 1e-4 of 2^x over the range the kernels use and
    returns exact zeros for masked (-inf) inputs."""
    import os
    import re
    import numpy as np
    src = open(os.path.join(os.path.dirname(__file__), "..", "chronicals_b200", "csrc", "common.cuh")).read()
    body = src[src.index("float ex2_fma(float x)"):]
    body = body[:body.index("\n}\n")]
    c3, c2 = [np.float32(v) for v in re.search(r"fmaf\(([0-9.]+)f, f, ([0-9.]+)f\)", body).groups()]
    c1, c0 = [np.float32(v) for v in re.findall(r"fmaf\(p, f, ([0-9.]+)f\)", body)]
    magic = np.float32(12582912.0)
    assert "12582912.f" in body and "<< 23" in body

    def ex2_fma(x):
        x = x.astype(np.float32)
        xc = np.maximum(x, np.float32(-125))
        t = (xc + magic).astype(np.float32)
        f = (xc - (t - magic).astype(np.float32)).astype(np.float32)
        p = (c3 * f + c2).astype(np.float32)
        p = (p * f + c1).astype(np.float32)
        p = (p * f + c0).astype(np.float32)
        bits = (p.view(np.int32).astype(np.int64) + ((t.view(np.int32).astype(np.int64) << 23) & 0xffffffff)) & 0xffffffff
        r = bits.astype(np.uint32).view(np.float32)
        return np.where(x < -125, np.float32(0), r)

    xs = np.linspace(-124.9, 9.5, 100001).astype(np.float32)
    err = np.abs(ex2_fma(xs) / np.exp2(xs.astype(np.float64)) - 1).max()
    assert err < 1e-4, err
    assert (ex2_fma(np.array([-np.inf, -300.0, -125.5], dtype=np.float32)) == 0).all()


def test_attention_tile_schedule_properties():
    """The attention kernels hand out tiles (128-row blocks of documents) by descending weight over all documents
    (``locate_tile`` in ``csrc/attention.cu``) and let the CTAs past the last tile zero the padding rows.  The same
    enumeration restated in Python: every block of every document appears exactly once, weights never increase,
    and the grid ``ceil(T / 128) + n_docs`` always leaves enough CTAs past the last tile to cover the padding."""
    import random

    def locate_tile(cu, b):
        nb = [(cu[i + 1] - cu[i] + 127) >> 7 for i in range(len(cu) - 1)]
        for level in range(max(nb, default=0), 0, -1):
            docs = [d for d, n in enumerate(nb) if n >= level]          # document order
            if b < len(docs):
                return docs[b], level
            b -= len(docs)
        return None, b                                                  # index among the CTAs past the last tile

    rng = random.Random(0)
    for _ in range(200):
        n_docs = rng.randint(1, 70)
        lens = [rng.choice([0, 1, 63, 64, 65, 127, 128, 129, 300, 1024, 2500]) for _ in range(n_docs)]
        cu = [0]
        for length in lens:
            cu.append(cu[-1] + length)
        T = cu[-1] + rng.choice([0, 1, 127, 128, 500])
        grid_y = (T + 127) // 128 + n_docs
        seen, weights, beyond = set(), [], 0
        for b in range(grid_y):
            doc, w = locate_tile(cu, b)
            if doc is None:
                assert w == beyond                                        # consecutive indices past the last tile
                beyond += 1
                continue
            assert beyond == 0, "tiles come first"
            nblk = (lens[doc] + 127) >> 7
            assert 1 <= w <= nblk
            seen.add((doc, w))                                            # forward: q block w - 1; backward: kv block nblk - w
            weights.append(w)
        assert len(seen) == len(weights) == sum((length + 127) >> 7 for length in lens)
        assert weights == sorted(weights, reverse=True)
        assert beyond * 128 >= T - cu[-1], "CTAs past the last tile cover the padding rows"
