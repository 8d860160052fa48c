"""Numerics of every CUDA kernel against a plain PyTorch fp32 statement of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from astrai_b200.ops import native

    native.require()
    yield
    assert native.kernel_status("cuda") == 0, "a kernel recorded an expired bounded wait"


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize("a_k", [True, False])
@pytest.mark.parametrize("b_k", [True, False])
@pytest.mark.parametrize("shape", [(256, 512, 192), (200, 264, 72), (128, 256, 64), (1024, 768, 2048), (8, 8, 8)])
def test_gemm_layouts(a_k, b_k, shape):
    from astrai_b200 import ops

    m, n, k = shape
    torch.manual_seed(0)
    a = torch.randn((m, k) if a_k else (k, m), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((n, k) if b_k else (k, n), device="cuda", dtype=torch.bfloat16)
    ref = (a.float() if a_k else a.float().t()) @ (b.float().t() if b_k else b.float())
    out = ops.gemm(a, b, a_kmajor=a_k, b_kmajor=b_k)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    assert _rel_err(out, ref) < 1e-2
    out32 = ops.gemm(a, b, a_kmajor=a_k, b_kmajor=b_k, out_f32=True)
    assert _rel_err(out32, ref) < 1e-5 * max(1, k ** 0.5)
    acc = torch.ones((m, n), device="cuda", dtype=torch.float32)
    ops.gemm(a, b, out=acc, a_kmajor=a_k, b_kmajor=b_k, out_f32=True, accumulate=True)
    assert _rel_err(acc, ref + 1) < 1e-5 * max(1, k ** 0.5)


def test_gemm_many_tiles_persistent():
    from astrai_b200 import ops

    torch.manual_seed(1)
    a = torch.randn(4096, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(3072, 512, device="cuda", dtype=torch.bfloat16)
    out = ops.gemm(a, b)  # 32 x 12 = 384 tiles > 148 CTAs: every CTA loops, both TMEM buffers cycle
    assert _rel_err(out, a.float() @ b.float().t()) < 1e-2


def test_linear_autograd_matches_fp32():
    from astrai_b200 import ops

    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    y = ops.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(w.grad, wr.grad) < 1e-2


def test_linear_main_grad_accumulates_in_fp32():
    from astrai_b200 import ops

    torch.manual_seed(3)
    x = torch.randn(512, 128, device="cuda", dtype=torch.bfloat16)
    w = torch.nn.Parameter((torch.randn(256, 128, device="cuda") * 0.05).to(torch.bfloat16))
    w.main_grad = torch.zeros(256, 128, device="cuda", dtype=torch.float32)
    for _ in range(2):
        ops.linear(x, w).sum().backward()
    assert w.grad is None
    ref = 2 * torch.ones(512, 256, device="cuda").t() @ x.float()
    assert _rel_err(w.main_grad, ref) < 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("cols", [2048, 4096, 64, 100])
def test_rmsnorm(dtype, cols):
    from astrai_b200 import ops

    torch.manual_seed(4)
    x = torch.randn(37, cols, device="cuda", dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dtype).requires_grad_()
    y = ops.rms_norm(x, w, 1e-6)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = torch.nn.functional.rms_norm(xr, (cols,), wr, 1e-6)
    yr.backward(g.float())
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel_err(y, yr) < tol and _rel_err(x.grad, xr.grad) < tol and _rel_err(w.grad, wr.grad) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rope_matches_reference_and_inverts(dtype):
    from astrai_b200 import ops
    from astrai_b200.models.layers import rope_table
    from astrai_b200.ops import reference

    torch.manual_seed(5)
    table = rope_table(64, 512).cuda()
    pos = torch.randint(0, 512, (3, 50), device="cuda")
    f = table[pos]
    x = torch.randn(3, 50, 6, 64, device="cuda", dtype=dtype, requires_grad=True)
    y = ops.rotary(x, f)
    ref = reference.rotary(x.detach().float(), f)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert (y.float() - ref).abs().max().item() < tol * 4
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    reference.rotary(xr, f).backward(g.float())
    assert (x.grad.float() - xr.grad).abs().max().item() < tol * 4


def test_qkv_rope_split():
    from astrai_b200 import ops
    from astrai_b200.models.layers import rope_table
    from astrai_b200.ops import reference

    torch.manual_seed(6)
    hq, hkv, d, t = 8, 2, 128, 70
    f = rope_table(d, 256).cuda()[torch.arange(t, device="cuda")]
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q, k, v = ops.qkv_rope(qkv, f, hq, hkv, d)
    r3 = qkv.detach().float().view(t, hq + 2 * hkv, d)
    assert (q.float() - reference.rotary(r3[:, :hq], f)).abs().max() < 5e-2
    assert (k.float() - reference.rotary(r3[:, hq:hq + hkv], f)).abs().max() < 5e-2
    assert torch.equal(v.float(), r3[:, hq + hkv:])
    (q.float().sum() + 2 * k.float().sum() + 3 * v.float().sum()).backward()
    assert qkv.grad is not None and torch.isfinite(qkv.grad.float()).all()
    assert torch.allclose(qkv.grad.float().view(t, -1, d)[:, hq + hkv:], torch.full((t, hkv, d), 3.0, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu(dtype):
    from astrai_b200 import ops

    torch.manual_seed(7)
    gu = torch.randn(33, 2 * 688, device="cuda", dtype=dtype, requires_grad=True)
    y = ops.swiglu_fused(gu)
    g = torch.randn_like(y)
    y.backward(g)
    r = gu.detach().float().requires_grad_()
    yr = r[:, 688:] * torch.nn.functional.silu(r[:, :688])
    yr.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel_err(y, yr) < tol and _rel_err(gu.grad, r.grad) < tol
    a = torch.randn(5, 7, 64, device="cuda", dtype=dtype)
    b = torch.randn(5, 7, 64, device="cuda", dtype=dtype)
    assert _rel_err(ops.swiglu(a, b), b.float() * torch.nn.functional.silu(a.float())) < tol


def test_embedding_forward_backward():
    from astrai_b200 import ops

    torch.manual_seed(8)
    table = torch.randn(1000, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 1000, (4, 33), device="cuda")
    out = ops.embedding(ids, table)
    assert torch.equal(out, table.detach()[ids])
    g = torch.randn_like(out)
    out.backward(g)
    ref = torch.zeros(1000, 64, device="cuda").index_add_(0, ids.reshape(-1), g.float().reshape(-1, 64))
    assert _rel_err(table.grad, ref) < 1e-2


@pytest.mark.parametrize("smoothing", [0.0, 0.05])
@pytest.mark.parametrize("vocab", [32000, 1003])
def test_linear_cross_entropy(smoothing, vocab):
    from astrai_b200 import ops

    torch.manual_seed(9)
    t, d = 300, 256
    h = torch.randn(t, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(vocab, d, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    tgt = torch.randint(0, vocab, (t,), device="cuda")
    tgt[::7] = -100
    loss = ops.linear_cross_entropy(h, w, tgt, smoothing, -100, chunk_tokens=128)
    (loss * 0.5).backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = torch.nn.functional.cross_entropy(hr @ wr.t(), tgt, label_smoothing=smoothing, ignore_index=-100)
    (lr * 0.5).backward()
    assert abs(loss.item() - lr.item()) < 2e-2
    assert _rel_err(h.grad, hr.grad) < 3e-2 and _rel_err(w.grad, wr.grad) < 3e-2


def test_linear_token_logprobs():
    from astrai_b200 import ops

    torch.manual_seed(10)
    h = torch.randn(2, 40, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(777, 128, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    ids = torch.randint(0, 777, (2, 40), device="cuda")
    lp = ops.linear_token_logprobs(h, w, ids, chunk_tokens=32)
    g = torch.randn_like(lp)
    lp.backward(g)
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = torch.log_softmax(hr @ wr.t(), -1).gather(-1, ids.unsqueeze(-1)).squeeze(-1)
    ref.backward(g)
    assert (lp - ref).abs().max().item() < 3e-2
    assert _rel_err(h.grad, hr.grad) < 3e-2 and _rel_err(w.grad, wr.grad) < 3e-2


def test_adamw_matches_torch():
    from astrai_b200 import ops

    torch.manual_seed(11)
    n = 100003
    p0 = torch.randn(n, device="cuda")
    p = p0.to(torch.bfloat16)
    master = p.float().clone()
    ref = torch.nn.Parameter(master.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref.grad = g.clone()
        opt.step()
        ops.adamw_(p, g, m, v, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, step=step, master=master, zero_grad=True)
        assert g.abs().sum().item() == 0
    assert (master - ref.detach()).abs().max().item() < 1e-5
    assert torch.equal(p, master.to(torch.bfloat16))


def test_sumsq_and_clip():
    from astrai_b200 import ops

    torch.manual_seed(12)
    x = torch.randn(1 << 20, device="cuda")
    s = ops.sumsq(x)
    assert abs(s.item() / x.double().pow(2).sum().item() - 1) < 1e-4
    coef, norm = ops.clip_coef(s, 1.0, 0.5)
    ref_norm = x.double().norm().item() * 0.5
    assert abs(norm.item() / ref_norm - 1) < 1e-4
    assert abs(coef.item() - min(1.0, 1.0 / (ref_norm + 1e-6)) * 0.5) < 1e-6


@pytest.mark.parametrize("hd,hq,hkv", [(128, 16, 4), (64, 8, 8), (256, 4, 1), (32, 8, 2), (64, 24, 4), (128, 6, 2), (64, 5, 1)])
@pytest.mark.parametrize("lens", [[1, 17, 300, 2049], [513]])
def test_paged_decode_matches_fp32(hd, hq, hkv, lens):
    torch.manual_seed(13)
    b, page, max_ctx = len(lens), 16, 2304
    n_slots = 4096
    k_buf = torch.randn(n_slots, hkv, hd, device="cuda", dtype=torch.bfloat16)
    v_buf = torch.randn(n_slots, hkv, hd, device="cuda", dtype=torch.bfloat16)
    table = torch.zeros(b + 1, max_ctx, dtype=torch.int32, device="cuda")
    perm = torch.randperm(n_slots // page, device="cuda")
    used = 0
    rows = torch.arange(b, dtype=torch.int32, device="cuda").flip(0).contiguous()  # request i lives in table row b-1-i
    for i, n in enumerate(lens):
        pages = perm[used:used + -(-n // page)]
        used += pages.numel()
        slots = (pages[:, None] * page + torch.arange(page, device="cuda")[None]).reshape(-1)[:n]
        table[rows[i], :n] = slots.int()
    q = torch.randn(b, hq, hd, device="cuda", dtype=torch.bfloat16)
    seq = torch.tensor(lens, dtype=torch.long, device="cuda")
    o_part = torch.zeros(b, hq, 32, hd, device="cuda")
    ml_part = torch.zeros(b, hq, 32, 2, device="cuda")
    counters = torch.zeros(b * hkv, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    for splits in (1, 5, 32):
        torch.ops.astrai_b200.paged_decode_(q, k_buf, v_buf, table, rows, seq, hd ** -0.5, splits, o_part, ml_part, counters, out)
        assert counters.sum().item() == 0  # self-resetting: ready for a graph replay
        for i, n in enumerate(lens):
            slots = table[rows[i], :n].long()
            k = k_buf[slots].float().repeat_interleave(hq // hkv, dim=1)
            v = v_buf[slots].float().repeat_interleave(hq // hkv, dim=1)
            att = torch.softmax(torch.einsum("hd,nhd->hn", q[i].float(), k) * hd ** -0.5, dim=-1)
            ref = torch.einsum("hn,nhd->hd", att, v)
            assert (out[i].float() - ref).abs().max().item() < 2e-2, (splits, i)


def test_kv_append_scatter():
    torch.manual_seed(14)
    k_buf = torch.zeros(64, 2, 64, device="cuda", dtype=torch.bfloat16)
    v_buf = torch.zeros_like(k_buf)
    k = torch.randn(5, 2, 64, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(5, 2, 64, device="cuda", dtype=torch.bfloat16)
    loc = torch.tensor([3, 60, 0, 17, 999], dtype=torch.int32, device="cuda")  # the last slot is out of range: skipped
    torch.ops.astrai_b200.kv_append_(k, v, k_buf, v_buf, loc)
    assert torch.equal(k_buf[[3, 60, 0, 17]], k[:4]) and torch.equal(v_buf[[3, 60, 0, 17]], v[:4])
    assert k_buf.float().abs().sum().item() == pytest.approx(k[:4].float().abs().sum().item(), rel=1e-3)


def test_engine_on_gpu_graph_replay_matches_eager(tmp_path):
    import sys

    sys.path.insert(0, str(__import__("pathlib").Path(__file__).parent))
    from helpers import build_tokenizer_dir

    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.inference import InferenceScheduler
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.tokenize import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(build_tokenizer_dir(str(tmp_path)))
    cfg = AutoRegressiveLMConfig(vocab_size=1024, hidden_size=256, num_hidden_layers=2, rms_norm_eps=1e-6, intermediate_size=512,
                                 tie_word_embeddings=True, max_position_embeddings=256, rope_theta=10000.0,
                                 num_attention_heads=4, num_key_value_heads=2)
    torch.manual_seed(0)
    model = AutoRegressiveLM(cfg).to("cuda", torch.bfloat16).eval()
    prompts = [list(range(5, 45)), list(range(100, 117)), list(range(5, 45)) + [77, 78]]
    eager = InferenceScheduler(model, tok, max_batch_size=4, max_seq_len=256, enable_cuda_graph=False)
    ref = eager.run_batch(prompts, max_tokens=12, temperature=0.0)
    graphed = InferenceScheduler(model, tok, max_batch_size=4, max_seq_len=256, enable_cuda_graph=True)
    assert graphed.cuda_graph_enabled
    got = graphed.run_batch(prompts, max_tokens=12, temperature=0.0)
    assert got == ref
    assert graphed.run_batch(prompts, max_tokens=12, temperature=0.0) == ref  # prefix-cache hit path, replayed graphs
    full = torch.tensor([prompts[1] + ref[1][:-1]], device="cuda")
    with torch.no_grad():
        logits = model(full)["logits"][0, len(prompts[1]) - 1:].float()
    agree = (logits.argmax(-1).tolist() == ref[1])
    assert agree or sum(a == b for a, b in zip(logits.argmax(-1).tolist(), ref[1])) >= 10  # bf16 near-ties may flip


def test_padded_decode_graph_buckets_match_eager(tmp_path):
    """Nine requests of different lengths decode on the 16-row graph (seven padded rows of length 0), five requests on the
    8-row graph; every token equals the eager run."""
    import sys

    sys.path.insert(0, str(__import__("pathlib").Path(__file__).parent))
    from helpers import build_tokenizer_dir

    from astrai_b200.config import AutoRegressiveLMConfig
    from astrai_b200.inference import InferenceScheduler
    from astrai_b200.inference.runtime.executor import Executor
    from astrai_b200.models import AutoRegressiveLM
    from astrai_b200.tokenize import AutoTokenizer

    assert Executor.decode_buckets(128) == [1, 2, 4, 8, 16, 24, 32, 40, 48, 56, 64, 80, 96, 112, 128]
    assert Executor.decode_buckets(12) == [1, 2, 4, 8, 12]
    tok = AutoTokenizer.from_pretrained(build_tokenizer_dir(str(tmp_path)))
    cfg = AutoRegressiveLMConfig(vocab_size=1024, hidden_size=256, num_hidden_layers=2, rms_norm_eps=1e-6, intermediate_size=512,
                                 tie_word_embeddings=True, max_position_embeddings=256, rope_theta=10000.0,
                                 num_attention_heads=4, num_key_value_heads=2)
    torch.manual_seed(3)
    model = AutoRegressiveLM(cfg).to("cuda", torch.bfloat16).eval()
    prompts = [list(range(10 + 7 * i, 10 + 7 * i + 5 + 9 * i)) for i in range(9)]
    eager = InferenceScheduler(model, tok, max_batch_size=16, max_seq_len=256, enable_cuda_graph=False)
    ref = eager.run_batch(prompts, max_tokens=20, temperature=0.0)
    graphed = InferenceScheduler(model, tok, max_batch_size=16, max_seq_len=256, enable_cuda_graph=True)
    assert graphed._executor._buckets == [1, 2, 4, 8, 16]
    assert graphed.run_batch(prompts, max_tokens=20, temperature=0.0) == ref
    assert graphed.run_batch(prompts[:5], max_tokens=20, temperature=0.0) == ref[:5]  # bucket 8, three padded rows


@pytest.mark.parametrize("m,n,k", [(1, 2048, 2048), (16, 3072, 2048), (17, 2048, 5632), (64, 11264, 2048), (33, 32000, 2048), (5, 384, 200), (100, 3072, 2048), (256, 2048, 5632), (200, 11264, 2048)])
def test_skinny_gemm_matches_fp32(m, n, k):
    """Decode-sized batches take the split-K kernel with the weight as the MMA's M operand."""
    from astrai_b200 import ops
    from astrai_b200.ops import native

    torch.manual_seed(21)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    for _ in range(2):  # the second call reuses the workspace and the self-resetting tile counters
        y = ops.gemm(x, w)
        ref = x.float() @ w.float().t()
        assert (y.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item() + 1e-2
    assert native.kernel_status(x.device) == 0


@pytest.mark.parametrize("rows,cols", [(64, 2048), (37, 1536), (5, 512)])
def test_add_rms_norm_matches_unfused(rows, cols):
    """Residual add fused into the norm, forward and backward, against the fp32 statement of the two separate ops."""
    from astrai_b200 import ops

    torch.manual_seed(11)
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    s, y = ops.add_rms_norm(x, r, w, 1e-6)
    gs, gy = torch.randn_like(s), torch.randn_like(y)
    (s * gs).sum().backward(retain_graph=True)
    dx_s = x.grad.clone()
    x.grad = r.grad = w.grad = None
    ((s * gs).sum() + (y * gy).sum()).backward()
    xf, rf, wf = (t.detach().float().requires_grad_(True) for t in (x, r, w))
    sf = xf + rf
    sf = sf + (sf.to(torch.bfloat16).float() - sf).detach()  # value rounded as the kernel stores it, gradient of the plain sum
    yf = torch.nn.functional.rms_norm(sf, (cols,), wf, 1e-6)
    ((sf * gs.float()).sum() + (yf * gy.float()).sum()).backward()
    assert torch.equal(s, (x.detach().float() + r.detach().float()).to(torch.bfloat16))
    assert (y.float() - yf).abs().max().item() < 3e-2
    assert torch.equal(dx_s, gs)  # only the residual branch: the gradient passes through unchanged
    assert torch.equal(x.grad, r.grad)
    assert (x.grad.float() - xf.grad).abs().max().item() < 6e-2
    assert ((w.grad.float() - wf.grad).abs().max() / wf.grad.abs().max()).item() < 2e-2
