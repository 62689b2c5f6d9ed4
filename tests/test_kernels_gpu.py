"""CUDA kernels against plain PyTorch fp32 references of the same ops (tiny and odd shapes)."""
import math

import pytest
import torch

from chronicals_b200 import ops
from chronicals_b200.ops import _ext, ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _close(a, b, rtol=2e-2, atol=2e-2, what="", l2=1e-2):
    """Three bounds: the largest error against the largest magnitude, the relative L2 error of the whole tensor,
    and an element-wise bound on a random sample that scales with each element's own row (so rows or columns of
    small magnitude cannot hide behind large ones)."""
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref_mag = b.abs().max().item()
    assert err <= atol + rtol * ref_mag, f"{what}: max err {err:.4g} vs magnitude {ref_mag:.4g}"
    rel = ((a - b).norm() / b.norm().clamp_min(1e-30)).item()
    assert rel <= l2 or (a - b).abs().max().item() <= atol, f"{what}: relative L2 error {rel:.4g}"
    if b.dim() == 2 and b.numel() > 0:
        g = torch.Generator(device="cpu").manual_seed(1234)
        rows = torch.randint(0, b.shape[0], (min(64, b.shape[0]),), generator=g).to(b.device)
        row_mag = b[rows].abs().amax(dim=1, keepdim=True)
        bad = ((a[rows] - b[rows]).abs() > atol + 4 * rtol * row_mag).sum().item()
        assert bad == 0, f"{what}: {bad} sampled elements beyond their row's tolerance"


def test_library_loaded_and_status_clean():
    assert _ext.available()
    _ext.lib()
    _ext.check_status()


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (200, 136, 72), (8192, 1152, 896),
                                   (1000, 896, 4864), (130, 8, 64)])
@pytest.mark.parametrize("block_n", [0, 128, 256])
def test_gemm_forward_kk(M, N, K, block_n):
    a, b = _rand(M, K), _rand(N, K, seed=1)
    bias = _rand(N, seed=2)
    add = _rand(M, N, seed=3)
    y = ops.gemm(a, b, bias=bias, addend=add, block_n=block_n)
    want = a.float() @ b.float().t() + bias.float() + add.float()
    _close(y, want, rtol=1e-2, atol=1e-2 * math.sqrt(K), what=f"gemm kk {M}x{N}x{K} bn={block_n}")
    _ext.check_status()


@pytest.mark.parametrize("M,N,K", [(256, 128, 192), (8192, 896, 1152), (520, 264, 136)])
def test_gemm_dgrad_layout(M, N, K):
    # dX[M, N] = dY[M, K] @ W[K, N]  -> B operand stored [K, N] (N contiguous)
    dy, w = _rand(M, K), _rand(K, N, seed=1)
    y = ops.gemm(dy, w, b_mn=True)
    _close(y, dy.float() @ w.float(), rtol=1e-2, atol=1e-2 * math.sqrt(K), what="dgrad")
    _ext.check_status()


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (1152, 896, 8192), (264, 136, 520)])
def test_gemm_wgrad_layout(M, N, K):
    # dW[M, N] = dY[K, M]^T @ X[K, N]  -> both operands stored with K as the row index
    dy, x = _rand(K, M), _rand(K, N, seed=1)
    y = ops.gemm(dy, x, a_mn=True, b_mn=True)
    _close(y, dy.float().t() @ x.float(), rtol=1e-2, atol=1e-2 * math.sqrt(K), what="wgrad")
    y32 = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    ops.gemm(dy, x, a_mn=True, b_mn=True, out=y32)
    ops.gemm(dy, x, a_mn=True, b_mn=True, out=y32, accumulate=True)
    _close(y32, 2 * (dy.float().t() @ x.float()), rtol=1e-2, atol=2e-2 * math.sqrt(K), what="wgrad fp32 accumulate")
    _ext.check_status()


def test_linear_autograd_matches_torch():
    x = _rand(300, 256).requires_grad_()
    w = _rand(384, 256, scale=0.05, seed=1).requires_grad_()
    b = _rand(384, seed=2).requires_grad_()
    r = _rand(300, 384, seed=3).requires_grad_()
    y = ops.linear(x, w, b, r)
    g = _rand(300, 384, seed=4)
    y.backward(g)
    xr, wr, br, rr = (t.detach().float().requires_grad_() for t in (x, w, b, r))
    yr = torch.nn.functional.linear(xr, wr, br) + rr
    yr.backward(g.float())
    _close(y, yr, what="linear fwd")
    _close(x.grad, xr.grad, what="linear dx")
    _close(w.grad, wr.grad, rtol=2e-2, atol=0.3, what="linear dw")
    _close(b.grad, br.grad, rtol=2e-2, atol=0.3, what="linear db")
    _close(r.grad, rr.grad, what="linear dres")


@pytest.mark.parametrize("M,N", [(64, 896), (1000, 3584), (77, 5120), (16, 256), (33, 8192)])
def test_rmsnorm_fwd_bwd(M, N):
    x = _rand(M, N).requires_grad_()
    w = (1 + 0.1 * _rand(N, seed=1).float()).to(torch.bfloat16).requires_grad_()
    y = ops.rmsnorm(x, w, 1e-6)
    g = _rand(M, N, seed=2)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.rmsnorm(xr, wr, 1e-6)
    yr.backward(g.float())
    _close(y, yr, what="rmsnorm fwd")
    _close(x.grad, xr.grad, what="rmsnorm dx")
    _close(w.grad, wr.grad, rtol=2e-2, atol=0.05 * math.sqrt(M), what="rmsnorm dw")


def test_add_rmsnorm_fused_residual():
    x, r = _rand(130, 896).requires_grad_(), _rand(130, 896, seed=1).requires_grad_()
    w = _rand(896, seed=2).requires_grad_()
    y, h = ops.add_rmsnorm(x, r, w)
    (y.float().sum() + 2 * h.float().sum()).backward()
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    hr = (xr + rr).to(torch.bfloat16).float()
    yr = ref.rmsnorm(xr + rr, wr)
    (yr.sum() + 2 * (xr + rr).sum()).backward()
    _close(h, hr, what="residual sum")
    _close(y, yr, what="add_rmsnorm fwd")
    _close(x.grad, xr.grad, what="add_rmsnorm dx")
    _close(r.grad, rr.grad, what="add_rmsnorm dres")


@pytest.mark.parametrize("fn,reff", [(ops.swiglu, ref.swiglu_packed), (ops.geglu, ref.geglu_packed)])
def test_glu_fwd_bwd(fn, reff):
    gu = _rand(257, 2 * 688).requires_grad_()
    y = fn(gu)
    g = _rand(257, 688, seed=1)
    y.backward(g)
    gur = gu.detach().float().requires_grad_()
    yr = reff(gur)
    yr.backward(g.float())
    _close(y, yr, what="glu fwd")
    _close(gu.grad, gur.grad, what="glu bwd")


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("hq,hk,d", [(14, 2, 64), (5, 1, 128)])
def test_qk_rope_in_place_and_inverse(interleaved, hq, hk, d):
    T = 300
    qkv = _rand(T, (hq + 2 * hk) * d)
    cos, sin = ref.rope_cache(512, d, 1e6, device=DEV)
    pos = (torch.arange(T, device=DEV) % 97).long()
    orig = qkv.clone()
    out = ops.qk_rope_(qkv.clone().requires_grad_(False), cos, sin, pos, hq, hk, d, interleaved)
    q = orig[:, :hq * d].view(T, hq, d)
    k = orig[:, hq * d:(hq + hk) * d].view(T, hk, d)
    qr = ref.apply_rope(q.float(), cos, sin, pos, interleaved)
    kr = ref.apply_rope(k.float(), cos, sin, pos, interleaved)
    _close(out[:, :hq * d], qr.reshape(T, -1), what="rope q")
    _close(out[:, hq * d:(hq + hk) * d], kr.reshape(T, -1), what="rope k")
    assert torch.equal(out[:, (hq + hk) * d:], orig[:, (hq + hk) * d:]), "V must be untouched"
    # backward = inverse rotation
    x = orig.clone().requires_grad_()
    y = ops.qk_rope_(x * 1.0, cos, sin, pos, hq, hk, d, interleaved)
    y.backward(out.detach())
    _close(x.grad[:, :hq * d], orig[:, :hq * d], what="rope inverse")


def test_embedding_fwd_bwd_deterministic():
    V, N, T = 1000, 896, 4096
    table = _rand(V, N).requires_grad_()
    ids = torch.randint(0, V, (T,), device=DEV)
    ids[:100] = 7                     # a long run of one id
    y = ops.embedding(ids, table)
    assert torch.equal(y, table.detach()[ids])
    g = _rand(T, N, seed=1)
    y.backward(g)
    want = torch.zeros(V, N, device=DEV).index_add_(0, ids, g.float())
    _close(table.grad, want, rtol=1e-2, atol=0.1, what="embedding bwd")
    g1 = table.grad.clone()
    table.grad = None
    ops.embedding(ids, table).backward(g)
    assert torch.equal(g1, table.grad), "scatter-add must be run-to-run deterministic"


@pytest.mark.parametrize("T,H,V", [(256, 256, 4096), (300, 896, 5000), (128, 64, 520)])
@pytest.mark.parametrize("smoothing,z", [(0.0, 0.0), (0.1, 1e-4)])
@pytest.mark.parametrize("resident", [False, True])
def test_linear_cross_entropy_fwd_bwd(T, H, V, smoothing, z, resident, monkeypatch):
    """Both forms: logits never held (online log-sum-exp in the GEMM epilogue, chunked recomputation in the
    backward pass) and logits resident in bf16 between forward and backward."""
    monkeypatch.setattr(ops, "CCE_RESIDENT_BYTES", (1 << 40) if resident else 0)
    h = _rand(T, H).requires_grad_()
    w = _rand(V, H, scale=0.05, seed=1).requires_grad_()
    y = torch.randint(0, V, (T,), device=DEV)
    y[::7] = -100
    loss = ops.linear_cross_entropy(h, w, y, None, -100, smoothing, z)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr_ = ref.linear_cross_entropy_dense(hr, wr, y, None, -100, smoothing, z)
    lr_.backward()
    assert abs(loss.item() - lr_.item()) < 2e-3 * max(1.0, abs(lr_.item())), (loss.item(), lr_.item())
    _close(h.grad, hr.grad, rtol=3e-2, atol=1e-5, what="cce dh")
    _close(w.grad, wr.grad, rtol=3e-2, atol=1e-5, what="cce dw")
    _ext.check_status()


@pytest.mark.parametrize("V", [32000, 151936])
@pytest.mark.parametrize("resident", [False, True])
def test_linear_cross_entropy_full_vocabularies_against_fp32(V, resident, monkeypatch):
    """The vocabulary sizes of the benchmark configurations (4 and 38 splits of the forward, 4 and 19 chunks of the
    backward), a token count that is not a multiple of the tile, labels in the first and last vocabulary rows;
    with and without resident logits."""
    monkeypatch.setattr(ops, "CCE_RESIDENT_BYTES", (1 << 40) if resident else 0)
    T, H = 200, 256
    h = _rand(T, H).requires_grad_()
    w = _rand(V, H, scale=0.05, seed=1).requires_grad_()
    y = torch.randint(0, V, (T,), device=DEV)
    y[0], y[1], y[2] = 0, V - 1, -100
    loss = ops.linear_cross_entropy(h, w, y, None, -100, 0.0, 1e-4)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    want = ref.linear_cross_entropy_dense(hr, wr, y, None, -100, 0.0, 1e-4)
    want.backward()
    assert abs(loss.item() - want.item()) < 2e-3 * max(1.0, abs(want.item())), (loss.item(), want.item())
    _close(h.grad, hr.grad, rtol=3e-2, atol=1e-5, what="cce dh", l2=2e-2)
    rel = ((w.grad.float() - wr.grad).norm() / wr.grad.norm()).item()
    assert rel < 2e-2, rel
    # the label rows carry the largest weight gradients: check them element by element
    rows = y[y >= 0].unique()
    _close(w.grad[rows], wr.grad[rows], rtol=3e-2, atol=1e-6, what="cce dw label rows", l2=2e-2)
    _ext.check_status()


@pytest.mark.parametrize("M,K,I,bias", [(300, 896, 4864, False), (513, 128, 256, True), (64, 64, 192, False)])
def test_linear_swiglu_in_the_projection_epilogue(M, K, I, bias, monkeypatch):
    """silu(gate) * up written by the gate | up GEMM's epilogue: agrees with the projection followed by the
    stand-alone activation kernel to bf16 rounding (both start from gate and up rounded to bf16; the epilogue
    evaluates the sigmoid through tanh.approx), same gradients; checked against fp32.
    I = 192 is not a multiple of the 128-column tile and takes the two-kernel path."""
    x = _rand(M, K).requires_grad_()
    w = (_rand(2 * I, K, seed=1) * 0.05).requires_grad_()
    b = (_rand(2 * I, seed=2) * 0.1).requires_grad_() if bias else None
    monkeypatch.setattr(ops, "_FUSED_GLU", "2")              # the fused kernel even where the environment turned it off
    act = ops.linear_swiglu(x, w, b)
    g = _rand(M, I, seed=3)
    act.backward(g)
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    b2 = b.detach().clone().requires_grad_() if bias else None
    two = ops.swiglu(ops.linear(x2, w2, b2))
    two.backward(g)
    _close(act, two, rtol=8e-3, atol=1e-3, what="linear_swiglu fused vs two-kernel activation", l2=4e-3)
    _close(x.grad, x2.grad, rtol=1e-2, atol=1e-3, what="linear_swiglu dx vs two-kernel path")
    _close(w.grad, w2.grad, rtol=1e-2, atol=1e-3, what="linear_swiglu dw vs two-kernel path")
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    br = b.detach().float().requires_grad_() if bias else None
    gu = torch.nn.functional.linear(xr, wr, br)
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    want.backward(g.float())
    _close(act, want, what="linear_swiglu fwd")
    _close(x.grad, xr.grad, rtol=3e-2, atol=3e-2, what="linear_swiglu dx")
    _close(w.grad, wr.grad, rtol=3e-2, atol=3e-2, what="linear_swiglu dw")
    if bias:
        _close(b.grad, br.grad, rtol=3e-2, atol=3e-2, what="linear_swiglu dbias")
    _ext.check_status()


def test_cross_entropy_logits_kernel():
    lg = _rand(200, 3000, dtype=torch.float32).requires_grad_()
    y = torch.randint(0, 3000, (200,), device=DEV)
    y[::5] = -100
    loss = ops.cross_entropy_logits(lg, y, -100, 0.1, 1e-4)
    loss.backward()
    lr_ = lg.detach().clone().requires_grad_()
    want = ref.cross_entropy_logits(lr_, y, -100, 0.1, 1e-4)
    want.backward()
    assert abs(loss.item() - want.item()) < 1e-4
    _close(lg.grad, lr_.grad, rtol=1e-3, atol=1e-7, what="ce grad")


@pytest.mark.parametrize("hq,hk,d", [(14, 2, 64), (4, 4, 64), (5, 1, 128)])
@pytest.mark.parametrize("bounds,T", [([0, 130, 131, 400, 640], 768), ([0, 1024], 768), ([0, 128, 256, 700], 768),
                                      ([0, 57, 301, 555], 555)])
def test_attention_packed_fwd_bwd(hq, hk, d, bounds, T):
    nq, nk = hq * d, hk * d
    qkv = _rand(T, nq + 2 * nk).requires_grad_()
    cu = torch.tensor([min(b, T) for b in bounds], dtype=torch.int32, device=DEV)
    valid = int(cu[-1].item())
    o = ops.attention_qkv_packed(qkv, cu, hq, hk, d)
    g = _rand(T, nq, seed=5)
    o.backward(g)
    xr = qkv.detach().float().requires_grad_()
    q = xr[:, :nq].reshape(T, hq, d)
    k = xr[:, nq:nq + nk].reshape(T, hk, d)
    v = xr[:, nq + nk:].reshape(T, hk, d)
    want = ref.attention_varlen(q, k, v, cu, None).reshape(T, nq)
    want.backward(g.float())
    _close(o[:valid], want[:valid], what="attention fwd")
    if valid < T:
        assert o[valid:].abs().max().item() == 0, "padding rows must be zero"
    _close(qkv.grad[:, :nq], xr.grad[:, :nq], rtol=3e-2, atol=3e-2, what="attention dq")
    _close(qkv.grad[:, nq:nq + nk], xr.grad[:, nq:nq + nk], rtol=3e-2, atol=3e-2, what="attention dk")
    _close(qkv.grad[:, nq + nk:], xr.grad[:, nq + nk:], rtol=3e-2, atol=3e-2, what="attention dv")
    _ext.check_status()


def test_attention_many_documents_and_large_scores():
    """More than 32 documents of mixed lengths (the tile schedule votes over the documents 32 at a time) and
    scores with a large spread (the running reference maximum of the forward has to be raised and the output
    accumulator rescaled several times along a row)."""
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(1, 300, (41,), generator=g).tolist() + [700, 129, 128, 64, 65]
    T = sum(lens) + 37
    hq, hk, d = 6, 2, 64
    nq, nk = hq * d, hk * d
    qkv = (_rand(T, nq + 2 * nk) * 3.0).requires_grad_()
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    valid = int(cu[-1].item())
    o = ops.attention_qkv_packed(qkv, cu, hq, hk, d)
    gr = _rand(T, nq, seed=9)
    o.backward(gr)
    xr = qkv.detach().float().requires_grad_()
    q = xr[:, :nq].reshape(T, hq, d)
    k = xr[:, nq:nq + nk].reshape(T, hk, d)
    v = xr[:, nq + nk:].reshape(T, hk, d)
    want = ref.attention_varlen(q, k, v, cu, None).reshape(T, nq)
    want.backward(gr.float())
    _close(o[:valid], want[:valid], rtol=3e-2, atol=3e-2, what="attention fwd (41+5 documents, large scores)")
    assert o[valid:].abs().max().item() == 0
    _close(qkv.grad[:valid], xr.grad[:valid], rtol=5e-2, atol=5e-2, what="attention dqkv (large scores)")
    _ext.check_status()


def test_attention_varlen_separate_tensors():
    T, hq, hk, d = 700, 14, 2, 64
    q, k, v = _rand(T, hq, d), _rand(T, hk, d, seed=1), _rand(T, hk, d, seed=2)
    cu = torch.tensor([0, 130, 131, 400, 640], dtype=torch.int32, device=DEV)
    o = ops.attention_varlen(q, k, v, cu, 269)
    want = ref.attention_varlen(q.float(), k.float(), v.float(), cu, 269)
    _close(o[:640], want[:640], what="attention fwd")
    assert o[640:].abs().max().item() == 0, "padding rows must be zero"


def test_fused_adamw_matches_torch():
    from chronicals_b200.optimizers.fused_adamw import FusedAdamW
    torch.manual_seed(0)
    shapes = [(1000, 33), (77,), (8192, 8), (5,)]
    ps = [torch.nn.Parameter(torch.randn(*s, device=DEV).to(torch.bfloat16)) for s in shapes]
    qs = [torch.nn.Parameter(p.detach().float().clone()) for p in ps]
    o1 = FusedAdamW(ps, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, max_grad_norm=1.0)
    o2 = torch.optim.AdamW(qs, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01)
    for step in range(4):
        for p, q in zip(ps, qs):
            g = torch.randn_like(q)
            p.grad = g.to(torch.bfloat16)
            q.grad = p.grad.float()
        torch.nn.utils.clip_grad_norm_(qs, 1.0)
        o1.step()
        o2.step()
        for p, q in zip(ps, qs):                     # keep the fp32 twin on the bf16 trajectory
            q.data.copy_(q.data.to(torch.bfloat16).float())
    for p, q in zip(ps, qs):
        _close(p, q, rtol=1e-2, atol=1e-2, what="adamw params")
    m1 = o1.state[ps[0]]["exp_avg"]
    m2 = o2.state[qs[0]]["exp_avg"]
    _close(m1, m2, rtol=1e-3, atol=1e-5, what="adamw exp_avg")


def test_tiny_model_step_runs_and_graph_matches_eager():
    from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    losses = {}
    for graphs in (False, True):
        model = build_model(cfg, dtype=torch.bfloat16, device=DEV, seed=0)
        args = TrainingConfig(output_dir="/tmp/cb_gpu_test", gradient_accumulation_steps=1, learning_rate=1e-3,
                              lr_scheduler_type="constant", warmup_ratio=0.0, logging_steps=1000, save_steps=0,
                              use_gradient_checkpointing=False, fp8=False, visual_reporting=False,
                              use_cuda_graphs=graphs, use_sequence_packing=False, z_loss_weight=1e-4)
        args.log_jsonl = False
        tr = ChronicalsTrainer(model, args, None)
        g = torch.Generator().manual_seed(0)
        out = []
        for i in range(6):
            ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=g)
            out.append(tr.training_step({"input_ids": ids, "labels": ids}).item())
        losses[graphs] = out
        _ext.check_status()
    assert all(math.isfinite(x) for x in losses[False])
    assert losses[False][-1] < losses[False][0] + 0.5
    for a, b in zip(losses[False], losses[True]):
        assert abs(a - b) < 5e-2, (losses[False], losses[True])


# ---------------------------------------------------------------------------------------------- MXFP8
@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("shape", [(257, 896), (64, 4864), (3, 32)])
def test_mxfp8_quant_kernel_matches_reference(fmt, shape):
    """Block-scaled quantisation (32-element blocks, e8m0 scales): scales must be bit-exact, payloads may
    differ by at most one fp8 step where the fp32 division rounds differently, and the dequantised copy
    must equal scale * payload exactly."""
    from chronicals_b200.ops import ref
    from chronicals_b200.utils.fp8_utils import mxfp8_quantize
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(*shape, generator=g) * torch.exp(2.0 * torch.randn(shape[0], 1, generator=g))).to(torch.bfloat16).cuda()
    x[0, :32] = 0                                                     # an all-zero block
    q, s, d = mxfp8_quantize(x, fmt, want_dequantized=True)
    q_ref, s_ref = ref.mxfp8_quantize(x.cpu(), fmt)
    assert torch.equal(s.cpu(), s_ref), "e8m0 scales differ"
    deq = ref.mxfp8_dequantize(q.cpu(), s.cpu(), torch.float32)
    deq_ref = ref.mxfp8_dequantize(q_ref, s_ref, torch.float32)
    step = 2.0 ** -3 if fmt == "e4m3" else 2.0 ** -2                  # relative spacing of the format's mantissa
    tol = step * deq_ref.abs().clamp(min=1e-30)
    assert bool(((deq - deq_ref).abs() <= tol + 1e-30).all())
    assert (q.cpu().float() != q_ref.float()).float().mean().item() < 1e-3
    assert torch.equal(d.cpu().float(), deq.to(torch.bfloat16).float())


def test_fp8_linear_module_runs_kernels_and_matches_reference():
    from chronicals_b200.ops import ref
    from chronicals_b200.utils.fp8_utils import FP8Linear
    torch.manual_seed(0)
    lin = FP8Linear(256, 384, bias=True).cuda().to(torch.bfloat16)
    x = torch.randn(96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = lin(x)
    y.float().pow(2).mean().backward()
    want = ref.mxfp8_linear(x.detach().float().cpu(), lin.weight.detach().float().cpu(), lin.bias.detach().float().cpu())
    assert (y.float().cpu() - want).abs().max().item() < 0.06 * want.abs().max().item()
    assert x.grad is not None and lin.weight.grad is not None and torch.isfinite(lin.weight.grad.float()).all()


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (200, 136, 160), (256, 384, 1024), (1024, 640, 4096)])
@pytest.mark.parametrize("fmts", [("e4m3", "e4m3"), ("e5m2", "e4m3")])
@pytest.mark.parametrize("tile", [128, 192])
def test_block_scaled_mxfp8_gemm_matches_dequantised_fp32_product(M, N, K, fmts, tile):
    """``tcgen05.mma.kind::mxf8f6f4.block_scale``: fp8 bytes and packed e8m0 scales in, bf16 out, against
    the fp32 product of the dequantised operands.  The scales vary by row and by 32-element block, so a wrong
    lane / column / byte mapping of the scale atoms cannot pass; ragged M, N and K exercise the padding.
    ``tile`` 128 runs the single-CTA kernel, 192 the CTA-pair kernel (B scales packed per 192-row tile)."""
    from chronicals_b200.ops import ref
    from chronicals_b200.utils import fp8_utils as F8
    assert F8.block_scaled_available(), "block-scaled GEMM kernel missing from the extension"
    g = torch.Generator(device="cuda").manual_seed(5)
    fa = torch.float8_e5m2 if fmts[0] == "e5m2" else torch.float8_e4m3fn
    a = torch.randn(M, K, device="cuda", generator=g).to(fa)
    b = torch.randn(N, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
    sa = torch.randint(120, 134, (M, K // 32), device="cuda", generator=g, dtype=torch.uint8)
    sb = torch.randint(120, 134, (N, K // 32), device="cuda", generator=g, dtype=torch.uint8)
    bias = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16)
    y = F8.mxfp8_block_scaled_matmul(a.view(torch.uint8), F8.pack_mx_scales(sa), b.view(torch.uint8),
                                     F8.pack_mx_scales(sb, tile), bias, fmts[0], fmts[1], b_tile_rows=tile).float()
    want = ref.mxfp8_dequantize(a, sa) @ ref.mxfp8_dequantize(b, sb).t() + bias.float()
    assert (y - want).abs().max().item() < 6e-3 * want.abs().max().item()


def test_mxfp8_packed_quantiser_writes_the_scale_atoms():
    from chronicals_b200.ops import ref
    from chronicals_b200.utils import fp8_utils as F8
    x = torch.randn(200, 160, device="cuda", dtype=torch.bfloat16) * 3
    q_ref, s_ref = ref.mxfp8_quantize(x.float())
    for tile in (128, 192):
        q, sf = F8.mxfp8_quantize_packed(x, tile_rows=tile)
        assert torch.equal(sf, F8.pack_mx_scales(s_ref, tile))
        assert (q != q_ref.view(torch.uint8)).float().mean().item() < 1e-3


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("shape", [(64, 96), (512, 896), (1024, 4864)])
def test_mxfp8_dual_quantiser_row_and_transposed_copies(fmt, shape):
    """One read of x gives the copy with blocks along the last dimension and the transposed copy with blocks
    along the first: both against the PyTorch quantiser (scales bit-exact, payload within one rounding)."""
    from chronicals_b200.ops import ref
    from chronicals_b200.utils import fp8_utils as F8
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(*shape, generator=g) * torch.exp(torch.randn(shape[0], 1, generator=g))).to(torch.bfloat16).cuda()
    q_row, sf_row, q_col, sf_col = F8.mxfp8_quantize_dual(x, fmt, 128, 192)
    qr, sr = ref.mxfp8_quantize(x.float(), fmt)
    qc, sc = ref.mxfp8_quantize(x.float().t().contiguous(), fmt)
    assert torch.equal(sf_row, F8.pack_mx_scales(sr)) and torch.equal(sf_col, F8.pack_mx_scales(sc, 192))
    assert (q_row != qr.view(torch.uint8)).float().mean().item() < 1e-3
    assert (q_col != qc.view(torch.uint8)).float().mean().item() < 1e-3
    only_col = F8.mxfp8_quantize_dual(x, fmt, 128, 192, want_row=False)
    assert only_col[0] is None and torch.equal(only_col[2], q_col)


def test_fp8_linear_gradients_on_block_scaled_tensor_cores():
    """dX and dW of the MXFP8 linear (e5m2 gradients × e4m3 operands, block-scaled MMAs) against the bf16
    autograd result: quantisation noise only."""
    from chronicals_b200.utils.fp8_utils import FP8Linear
    torch.manual_seed(1)
    lin = FP8Linear(512, 384, bias=True).cuda().to(torch.bfloat16)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16)
    lin(x).backward(gy)
    xr = x.detach().float().requires_grad_(True)
    wr = lin.weight.detach().float().requires_grad_(True)
    (xr @ wr.t() + lin.bias.detach().float()).backward(gy.float())
    for got, want in ((x.grad, xr.grad), (lin.weight.grad, wr.grad)):
        rel = (got.float() - want).norm() / want.norm()
        assert rel.item() < 0.08, rel.item()
    assert (lin.bias.grad.float() - gy.float().sum(0)).abs().max().item() < 0.02 * gy.float().sum(0).abs().max().item()


def test_linear_weight_gradient_of_a_small_weight_uses_split_k_and_matches_fp32():
    """out x in = 256 x 384 over 4096 tokens: 6 output tiles, so the token range is split across CTAs and the
    partial tiles meet through TMA reduce-add; a ragged 200 x 136 output exercises the clipped boxes."""
    from chronicals_b200 import ops
    torch.manual_seed(0)
    for n_out, n_in in ((256, 384), (200, 136)):
        x = torch.randn(4096, n_in, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(4096, n_out, device="cuda", dtype=torch.bfloat16)
        dw = ops.wgrad(dy, x)
        want = dy.float().t() @ x.float()
        assert dw.dtype == torch.bfloat16 and dw.shape == (n_out, n_in)
        assert (dw.float() - want).abs().max().item() < 8e-3 * want.abs().max().item()
        w = torch.randn(n_out, n_in, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        ops.linear(x, w).backward(dy)
        assert (w.grad.float() - want).abs().max().item() < 8e-3 * want.abs().max().item()


def test_fused_lora_projection_with_dropout_stays_on_the_fused_path():
    """Adapter dropout keeps the single fused autograd node (dual-product forward, split-K adapter gradients): with
    the random stream fixed, output and gradients equal the plain formula evaluated with the same keep mask."""
    from collections import OrderedDict
    from chronicals_b200.lora import functional as lf
    from chronicals_b200.models.decoder import FusedLinear
    torch.manual_seed(0)
    T, K, p = 256, 256, 0.25
    fl = FusedLinear(K, OrderedDict(gate_proj=384, up_proj=384), bias=False, dtype=torch.bfloat16, device="cuda")
    with torch.no_grad():
        fl.weight.normal_(0, 0.05)
    fl.weight.requires_grad_(False)
    for s in fl.splits:
        fl.add_lora(s, 16, 32.0)
        with torch.no_grad():
            fl.lora_B[s].normal_(0, 0.05)
    fl.lora_dropout_p = p
    fl.train()
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    assert lf._fused_path_ok(fl, x)
    torch.manual_seed(123)
    y = fl(x)
    gy = torch.randn_like(y)
    y.backward(gy)
    torch.manual_seed(123)
    keep = (torch.rand_like(x, dtype=torch.float32) >= p).float() / (1 - p)
    xf = x.detach().float().requires_grad_(True)
    A = {s: fl.lora_A[s].detach().float().requires_grad_(True) for s in fl.splits}
    B = {s: fl.lora_B[s].detach().float().requires_grad_(True) for s in fl.splits}
    want = xf @ fl.weight.float().t() + torch.cat([fl.lora_scaling[s] * ((xf * keep) @ A[s].t()) @ B[s].t()
                                                   for s in fl.splits], dim=1)
    want.backward(gy.float())
    _close(y, want, rtol=2e-2, atol=2e-2, what="lora dropout fwd")
    _close(x.grad, xf.grad, rtol=2e-2, atol=2e-2, what="lora dropout dx")
    for s in fl.splits:
        _close(fl.lora_A[s].grad, A[s].grad, rtol=3e-2, atol=3e-2, what="dA")
        _close(fl.lora_B[s].grad, B[s].grad, rtol=3e-2, atol=3e-2, what="dB")
    assert fl.weight.grad is None
    _ext.check_status()


def test_fused_lora_pack_and_unpack_kernels_match_the_operator_path(monkeypatch):
    """A_cat / B_big built, and their gradients split per adapter, by the two small kernels give what the
    PyTorch-operator assembly gives (same GEMMs in between): output and input gradient bit for bit, the adapter
    gradients up to the summation order of the split-K GEMM."""
    from collections import OrderedDict
    from chronicals_b200.lora import functional as lf
    from chronicals_b200.models.decoder import FusedLinear
    out = {}
    for use_pack in (True, False):
        monkeypatch.setattr(lf, "_USE_PACK", use_pack)
        torch.manual_seed(0)
        fl = FusedLinear(256, OrderedDict(q=384, k=128, v=128), bias=True, dtype=torch.bfloat16, device=DEV)
        with torch.no_grad():
            fl.weight.normal_(0, 0.05)
        fl.weight.requires_grad_(False)
        for i, (name, r) in enumerate((("q", 16), ("k", 8), ("v", 16))):
            fl.add_lora(name, rank=r, alpha=2.0 * r + i)
            with torch.no_grad():
                fl.lora_B[name].normal_(0, 0.05)
        x = _rand(300, 256, seed=4).requires_grad_()
        y = fl(x)
        y.backward(_rand(300, 640, seed=5))
        out[use_pack] = [y.detach(), x.grad] + [fl.lora_A[s].grad for s in ("q", "k", "v")] + [fl.lora_B[s].grad for s in ("q", "k", "v")]
    for i, (a, b) in enumerate(zip(out[True], out[False])):
        if i < 2:                                      # output and input gradient: same kernels on the same operands
            assert torch.equal(a, b), (i, (a.float() - b.float()).abs().max().item())
        else:                                          # adapter gradients pass a split-K sum whose order is not fixed
            _close(a, b, rtol=1e-3, atol=1e-4, what=f"adapter gradient {i}", l2=1e-3)
    _ext.check_status()


def test_fused_lora_projection_matches_reference_formula():
    """Frozen fused QKV projection with rank-16 adapters on every split: forward, dX, dA, dB against the
    plain PEFT formula in fp32 (the base weight must receive no gradient)."""
    from collections import OrderedDict
    from chronicals_b200.models.decoder import FusedLinear
    torch.manual_seed(0)
    T, K = 384, 256
    fl = FusedLinear(K, OrderedDict(q_proj=256, k_proj=64, v_proj=64), bias=True, dtype=torch.bfloat16, device="cuda")
    with torch.no_grad():
        fl.weight.normal_(0, 0.05)
        fl.bias.normal_(0, 0.1)
    fl.weight.requires_grad_(False)
    fl.bias.requires_grad_(False)
    for s in fl.splits:
        fl.add_lora(s, 16, 32.0)
        with torch.no_grad():
            fl.lora_B[s].normal_(0, 0.05)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    res = torch.randn(T, fl.out_features, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = fl(x, res)
    gy = torch.randn_like(y)
    y.backward(gy)
    # fp32 oracle
    xf, rf = x.detach().float().requires_grad_(True), res.detach().float().requires_grad_(True)
    A = {s: fl.lora_A[s].detach().float().requires_grad_(True) for s in fl.splits}
    B = {s: fl.lora_B[s].detach().float().requires_grad_(True) for s in fl.splits}
    base = xf @ fl.weight.float().t() + fl.bias.float() + rf
    parts = [fl.lora_scaling[s] * (xf @ A[s].t()) @ B[s].t() for s in fl.splits]
    want = base + torch.cat(parts, dim=1)
    want.backward(gy.float())

    def close(a, b, tol):
        return (a.float() - b).abs().max().item() <= tol * (b.abs().max().item() + 1e-6)
    assert close(y, want.detach(), 2e-2)
    assert close(x.grad, xf.grad, 3e-2) and close(res.grad, rf.grad, 1e-2)
    for s in fl.splits:
        assert close(fl.lora_A[s].grad, A[s].grad, 3e-2), s
        assert close(fl.lora_B[s].grad, B[s].grad, 3e-2), s
    assert fl.weight.grad is None


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(48, 896, 8192, True, True), (1152, 48, 8192, True, True), (16, 16, 300, False, False),
                                             (200, 130, 4096, False, True)])
def test_gemm_splitk_matches_fp32(M, N, K, a_mn, b_mn):
    from chronicals_b200 import ops
    g = torch.Generator().manual_seed(3)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g).to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), generator=g).to(torch.bfloat16)
    # row pitches must be multiples of 8 elements for the TMA path
    if (a.shape[1] % 8) or (b.shape[1] % 8):
        pytest.skip("operand pitch not TMA-addressable")
    out = ops.gemm_splitk(a.cuda(), b.cuda(), a_mn=a_mn, b_mn=b_mn)
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    want = A @ B
    assert out.dtype == torch.float32
    assert (out.cpu() - want).abs().max().item() < 2e-3 * want.abs().max().item() + 1e-3


def test_rope_positions_beyond_table_are_clamped_not_read_out_of_bounds():
    """Positions outside the cos/sin tables use the last table row (no out-of-bounds read); the optional
    debug build would additionally record code 402."""
    from chronicals_b200 import ops
    from chronicals_b200.ops import _ext, ref
    T, hq, hk, d = 64, 2, 1, 64
    cos, sin = ref.rope_cache(32, d, 1e4, device="cuda")
    qkv = torch.randn(T, (hq + 2 * hk) * d, device="cuda", dtype=torch.bfloat16)
    pos = torch.arange(T, device="cuda")                      # half of them beyond the 32-row table
    out = ops.qk_rope_(qkv.clone(), cos, sin, pos, hq, hk, d)
    want = ops.qk_rope_(qkv.clone(), cos, sin, pos.clamp(max=31), hq, hk, d)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    compiled, code, _ = _ext.debug_word()
    assert (code == 402) if compiled else (code == 0)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(512, 768, 320), (300, 200, 136), (1000, 896, 1024)])
def test_gemm_cta_pair_kernel_matches_fp32(a_mn, b_mn, M, N, K):
    """The cta_group::2 kernel (256x256 tile per CTA pair), forced with block_n=2, in all four operand layouts,
    with ragged edges in M, N and K."""
    from chronicals_b200 import ops
    g = torch.Generator().manual_seed(5)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g).to(torch.bfloat16).cuda()
    b = torch.randn((K, N) if b_mn else (N, K), generator=g).to(torch.bfloat16).cuda()
    if a.shape[1] % 8 or b.shape[1] % 8:
        pytest.skip("operand pitch not TMA-addressable")
    out = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=2)
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    want = A @ B
    assert (out.float() - want).abs().max().item() < 1.5e-2 * want.abs().max().item()
    _ext.check_status()


def test_gemm_cta_pair_kernel_epilogues():
    from chronicals_b200 import ops
    g = torch.Generator().manual_seed(6)
    M, N, K = 520, 896, 1024
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=g).to(torch.bfloat16).cuda()
    res = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    want = a.float() @ w.float().t() + bias.float() + res.float()
    out = ops.gemm(a, w, bias=bias, addend=res, block_n=2)
    assert (out.float() - want).abs().max().item() < 1.5e-2 * want.abs().max().item()
    acc32 = torch.randn(M, N, generator=g).cuda()
    want2 = acc32 + a.float() @ w.float().t()
    ops.gemm(a, w, out=acc32, accumulate=True, block_n=2)
    assert (acc32 - want2).abs().max().item() < 2e-3 * want2.abs().max().item()
    acc16 = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    want3 = acc16.float() + a.float() @ w.float().t()
    ops.gemm(a, w, out=acc16, accumulate=True, block_n=2)
    assert (acc16.float() - want3).abs().max().item() < 1.5e-2 * want3.abs().max().item()
    _ext.check_status()


def _rel_l2(got, want):
    return ((got.float() - want).norm() / want.norm().clamp_min(1e-30)).item()


@pytest.mark.parametrize("a_mn,b_mn,M,N,K,bn", [
    (False, False, 8192, 896, 4864, 0),      # down projection forward: 128 tiles of 256 x 224 on 74 pairs
    (False, True, 8192, 896, 1152, 0),       # dgrad layout, tile width 224 with the B halves in two 64-column atoms
    (True, True, 4864, 896, 8192, 0),        # wgrad layout: 76 tiles, every pair continues its neighbour's tile
    (True, True, 896, 4864, 8192, 0),
    (False, False, 8192, 1152, 896, 192),    # QKV: tile width 192
    (False, False, 4000, 1000, 520, 256),    # ragged M, N and K, runs of a few k-blocks
    (False, False, 2304, 640, 2048, 224),    # tile width that does not divide N
])
def test_gemm_cta_pair_stream_k_matches_fp32_and_whole_tiles(a_mn, b_mn, M, N, K, bn):
    """Tiles cut along K across CTA pairs (fp32 partial sums added in the workspace, last arrival runs the epilogue)
    against the fp32 product and against the same kernel restricted to whole tiles; the workspace is clean again
    afterwards (a second launch gives the same bits)."""
    from chronicals_b200 import ops
    g = torch.Generator().manual_seed(11)
    a = (torch.randn((K, M) if a_mn else (M, K), generator=g) * 0.5).to(torch.bfloat16).cuda()
    b = (torch.randn((K, N) if b_mn else (N, K), generator=g) * 0.5).to(torch.bfloat16).cuda()
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    want = A @ B
    split = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair_flags=(bn << 8) | 2)
    whole = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair_flags=(bn << 8) | 1)
    again = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair_flags=(bn << 8) | 2)
    _ext.check_status()
    assert _rel_l2(split, want) < 4e-3 and _rel_l2(whole, want) < 4e-3
    assert (split.float() - want).abs().max().item() < 1.5e-2 * want.abs().max().item()
    # split tiles are summed in fp32 before the single rounding, like whole tiles: at most an ulp apart
    assert (split.float() - whole.float()).abs().max().item() <= 2.0 ** -7 * want.abs().max().item()
    assert torch.equal(split, again)


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(2048, 896, 1536, False, False), (1024, 1152, 2048, False, True),
                                              (896, 640, 4096, True, True)])
def test_gemm_result_does_not_depend_on_tiling_stage_count_or_work_order(M, N, K, a_mn, b_mn):
    """The same product through every schedule the dispatcher can pick: single-CTA tiles of 128 and 256 columns
    (6 and 4 pipeline stages), CTA-pair tiles of 256 / 224 / 192 columns, whole tiles and tiles cut along K.  All
    of them accumulate each output element over the full K in fp32 and round once, so they agree with the fp32
    product and, element by element, with each other to one bf16 rounding step."""
    g = torch.Generator().manual_seed(21)
    a = (torch.randn((K, M) if a_mn else (M, K), generator=g) * 0.5).to(torch.bfloat16).cuda()
    b = (torch.randn((K, N) if b_mn else (N, K), generator=g) * 0.5).to(torch.bfloat16).cuda()
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    want = A @ B
    outs = {"single128": ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=128),
            "single256": ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=256)}
    for bn in (256, 224, 192):
        outs[f"pair{bn}"] = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair_flags=(bn << 8) | 1)
        outs[f"pair{bn}_split"] = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair_flags=(bn << 8) | 2)
    _ext.check_status()
    mag = want.abs().max().item()
    base = outs["single128"].float()
    for name, o in outs.items():
        assert _rel_l2(o, want) < 4e-3, name
        assert (o.float() - base).abs().max().item() <= 2.0 ** -7 * mag, name


def test_gemm_cta_pair_stream_k_epilogues():
    """Bias, residual, accumulate (bf16 and fp32 outputs) on a shape whose tiles are split along K."""
    from chronicals_b200 import ops
    g = torch.Generator().manual_seed(12)
    M, N, K = 8192, 896, 2048
    a = (torch.randn(M, K, generator=g) * 0.3).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.3).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=g).to(torch.bfloat16).cuda()
    res = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    prod = a.float() @ w.float().t()
    out = ops.gemm(a, w, bias=bias, addend=res, pair_flags=2)
    want = prod + bias.float() + res.float()
    assert _rel_l2(out, want) < 4e-3
    acc32 = torch.randn(M, N, generator=g).cuda()
    want2 = acc32 + prod
    ops.gemm(a, w, out=acc32, accumulate=True, pair_flags=2)
    assert _rel_l2(acc32, want2) < 1e-3
    acc16 = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    want3 = acc16.float() + prod
    ops.gemm(a, w, out=acc16, accumulate=True, pair_flags=2)
    assert _rel_l2(acc16, want3) < 4e-3
    o32 = ops.gemm(a, w, out_dtype=torch.float32, pair_flags=2)
    assert _rel_l2(o32, prod) < 1e-3
    _ext.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_adamw8bit_kernel_matches_python_path(dtype):
    """Fused 8-bit AdamW (block-wise quantised moments) against the same optimizer run through the PyTorch
    formulas: identical quantisation codes up to one rounding step, parameters equal to bf16/fp32 tolerance."""
    from chronicals_b200.optimizers.optimizers_8bit import AdamW8bit
    torch.manual_seed(0)
    n = 256 * 37 + 100                                       # a ragged last block
    p0 = torch.randn(n, device="cuda").to(dtype)
    grads = [torch.randn(n, device="cuda").to(dtype) * (0.5 ** i) for i in range(4)]
    pk = torch.nn.Parameter(p0.clone())
    pr = torch.nn.Parameter(p0.clone())
    ok = AdamW8bit([pk], lr=1e-2, weight_decay=0.01, min_8bit_size=1)
    orf = AdamW8bit([pr], lr=1e-2, weight_decay=0.01, min_8bit_size=1)
    for g in grads:
        pk.grad, pr.grad = g.clone(), g.clone()
        ok.step()
        with _ext.force_reference():
            orf.step()
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-3
    assert (pk.float() - pr.float()).abs().max().item() < tol
    sk, sr = ok.state[pk], orf.state[pr]
    assert (sk["exp_avg"].int() - sr["exp_avg"].int()).abs().max().item() <= 2
    assert (sk["exp_avg_sq"].int() - sr["exp_avg_sq"].int()).abs().max().item() <= 2
    assert torch.allclose(sk["exp_avg_absmax"], sr["exp_avg_absmax"], rtol=2e-2, atol=1e-6)


def test_newton_schulz_on_tensor_cores_orthogonalises():
    from chronicals_b200.optimizers.optimizers import newton_schulz_orthogonalize
    torch.manual_seed(0)
    g = torch.randn(256, 896, device="cuda").to(torch.bfloat16)
    x = newton_schulz_orthogonalize(g, steps=5).float()
    want = newton_schulz_orthogonalize(g.float().cpu(), steps=5)
    assert (x.cpu() - want).abs().max().item() < 0.05 * want.abs().max().item() + 5e-3
    d = (x @ x.t()).diagonal()                                                 # squared row norms, 1 / 256 at the start
    assert d.min().item() > 10.0 / 256 and d.max().item() < 1.3               # pulled towards an orthonormal set of rows


@pytest.mark.parametrize("M,N,K", [(512, 768, 256), (300, 200, 144), (1024, 896, 4864)])
def test_fp8_tensor_core_gemm_matches_dequantised_fp32(M, N, K):
    """kind::f8f6f4 GEMM on CTA pairs: e4m3 operands with per-row scales; the oracle multiplies the exactly
    dequantised operands in fp32, so only the bf16 rounding of the output separates the two."""
    from chronicals_b200.utils.fp8_utils import fp8_rowwise_matmul, rowwise_quantize_e4m3
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(M, K, generator=g) * torch.exp(torch.randn(M, 1, generator=g))).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=g).to(torch.bfloat16).cuda()
    xq, xs = rowwise_quantize_e4m3(x)
    wq, ws = rowwise_quantize_e4m3(w)
    # the quantisation kernel against the PyTorch formula
    with _ext.force_reference():
        xq_ref, xs_ref = rowwise_quantize_e4m3(x)
    assert torch.allclose(xs, xs_ref, rtol=1e-6)
    assert (xq != xq_ref).float().mean().item() < 1e-3
    y = fp8_rowwise_matmul(xq, xs, wq, ws, bias)
    a = xq.view(torch.float8_e4m3fn).float() * xs[:, None]
    b = wq.view(torch.float8_e4m3fn).float() * ws[:, None]
    want = a @ b.t() + bias.float()
    assert (y.float() - want).abs().max().item() < 1e-2 * want.abs().max().item()
    # and the quantisation error against the unquantised product stays at the e4m3 level
    full = x.float() @ w.float().t() + bias.float()
    assert (y.float() - full).abs().max().item() < 0.12 * full.abs().max().item()
    _ext.check_status()


def test_fp8_rowwise_linear_module_trains():
    from chronicals_b200.utils.fp8_utils import FP8RowwiseLinear
    torch.manual_seed(0)
    lin = FP8RowwiseLinear(256, 384).cuda()
    x = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = lin(x)
    y.float().pow(2).mean().backward()
    assert y.shape == (128, 384) and x.grad is not None and lin.weight.grad is not None
    ref_y = torch.nn.functional.linear(x.detach(), lin.weight.detach(), lin.bias.detach())
    assert (y.float() - ref_y.float()).abs().max().item() < 0.1 * ref_y.float().abs().max().item()


@pytest.mark.parametrize("M,N", [(8192, 1152), (300, 896), (1, 64), (1000, 4864)])
def test_colsum_kernel(M, N):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    out = ops.colsum(x)
    want = x.float().sum(0)
    assert out.dtype == torch.bfloat16 and out.shape == (N,)
    assert (out.float() - want).abs().max().item() < 1e-2 * want.abs().max().item() + 1e-2
    view = x[:, : N // 2] if (N // 2) % 8 == 0 else x                      # a strided view (column slice)
    assert (ops.colsum(view).float() - view.float().sum(0)).abs().max().item() < 1e-2 * want.abs().max().item() + 1e-2
