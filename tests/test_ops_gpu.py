"""sm_100a kernels vs the fp32 PyTorch oracle (zorse_b200.ops.ref on CPU)."""
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from zorse_b200.ops import ref


@pytest.fixture(scope="module")
def k():
    from zorse_b200.ops import sm100

    sm100.lib()
    return sm100


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def _close(got, want, atol, rtol):
    got = got.float().cpu()
    want = want.float().cpu()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = (err > tol).float().mean().item()
    assert bad == 0.0, f"max err {err.max().item():.4g}, frac bad {bad:.4g}"


GEMM_SHAPES = [
    (128, 128, 64), (128, 256, 64), (256, 512, 256), (200, 136, 72), (1, 8, 8),
    (384, 1376, 512), (512, 512, 2048), (1000, 1000, 264),
]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_layouts(k, M, N, K, a_mn, b_mn, bn):
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operand needs a 16-byte aligned row stride")
    a = _rand(M, K, seed=1)
    b = _rand(N, K, seed=2)
    want = a.float() @ b.float().t()
    ad = (a.t().contiguous() if a_mn else a).cuda()
    bd = (b.t().contiguous() if b_mn else b).cuda()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    k.gemm(ad, bd, out, a_mn=a_mn, b_mn=b_mn, bn=bn)
    k.check_status()
    _close(out, want, atol=0.02 * math.sqrt(K), rtol=1e-2)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (300, 520, 200), (1024, 1280, 4096), (4096, 1024, 512)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_pair_kernel(k, M, N, K, a_mn, b_mn):
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operand needs a 16-byte aligned row stride")
    a = _rand(M, K, seed=1)
    b = _rand(N, K, seed=2)
    want = a.float() @ b.float().t()
    ad = (a.t().contiguous() if a_mn else a).cuda()
    bd = (b.t().contiguous() if b_mn else b).cuda()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    k.gemm(ad, bd, out, a_mn=a_mn, b_mn=b_mn, kernel="2cta")
    k.check_status()
    _close(out, want, atol=0.02 * math.sqrt(K), rtol=1e-2)
    acc = torch.ones(M, N, dtype=torch.float32, device="cuda")
    k.gemm(ad, bd, acc, a_mn=a_mn, b_mn=b_mn, kernel="2cta", accumulate=True)
    k.check_status()
    _close(acc, want + 1, atol=0.02 * math.sqrt(K), rtol=1e-2)


def test_gemm_epilogues(k):
    M, N, K = 300, 520, 192
    a, b = _rand(M, K, seed=3), _rand(N, K, seed=4)
    bias, res = _rand(N, seed=5), _rand(M, N, seed=6)
    base = a.float() @ b.float().t()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    k.gemm(a.cuda(), b.cuda(), out, bias=bias.cuda(), addend=res.cuda())
    _close(out, base + bias.float() + res.float(), atol=0.3, rtol=1e-2)
    # fp32 accumulate, twice
    acc = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    k.gemm(a.cuda(), b.cuda(), acc, accumulate=True)
    k.gemm(a.cuda(), b.cuda(), acc, accumulate=True)
    _close(acc, 2 * base, atol=0.05, rtol=2e-3)
    # bf16 accumulate
    acc16 = res.cuda().clone()
    k.gemm(a.cuda(), b.cuda(), acc16, accumulate=True)
    _close(acc16, base + res.float(), atol=0.3, rtol=1e-2)
    # gelu after bias
    k.gemm(a.cuda(), b.cuda(), out, bias=bias.cuda(), act="gelu")
    _close(out, torch.nn.functional.gelu(base + bias.float(), approximate="tanh"), atol=0.3, rtol=1e-2)
    k.check_status()


def test_gemm_large_vs_fp32(k):
    M, N, K = 1024, 2048, 4096
    a, b = _rand(M, K, seed=7, scale=0.5), _rand(N, K, seed=8, scale=0.5)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    k.gemm(a.cuda(), b.cuda(), out)
    k.check_status()
    want = a.double() @ b.double().t()
    _close(out, want, atol=0.15, rtol=1e-2)


CANDIDATES = os.environ.get("ZORSE_TEST_CANDIDATES") == "1"   # kernel versions not yet validated on hardware


@pytest.mark.parametrize("bwd_version", [1, 2])
@pytest.mark.parametrize("T,H", [(5, 512), (300, 4096), (64, 2048), (33, 5120), (1000, 4096)])
@pytest.mark.parametrize("ln", [False, True])
def test_norm(k, T, H, ln, bwd_version):
    x, w, b = _rand(T, H, seed=1), (_rand(H, seed=2) * 0.1 + 1).to(torch.bfloat16), _rand(H, seed=3, scale=0.1)
    dy, dres = _rand(T, H, seed=4), _rand(T, H, seed=5)
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    br = b.float().requires_grad_(True)
    if ln:
        yr = torch.nn.functional.layer_norm(xr, (H,), wr, br, 1e-5)
    else:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(dy.float())
    y, stats = k.norm_fwd(x.cuda(), w.cuda(), b.cuda() if ln else None, 1e-5, ln, version=bwd_version)
    _close(y, yr.detach(), atol=2e-2, rtol=1e-2)
    for gdt in (torch.float32, torch.bfloat16):
        dw = torch.ones(H, dtype=gdt, device="cuda")
        db = torch.ones(H, dtype=gdt, device="cuda")
        dx = k.norm_bwd(dy.cuda(), x.cuda(), w.cuda(), stats, dres.cuda(), dw, db if ln else None, ln,
                        version=bwd_version)
        _close(dx, xr.grad + dres.float(), atol=5e-2, rtol=2e-2)
        tol = 0.02 * math.sqrt(T) + (0.3 if gdt == torch.bfloat16 else 0)
        _close(dw, wr.grad + 1, atol=tol, rtol=2e-2)
        if ln:
            _close(db, br.grad + 1, atol=tol, rtol=2e-2)


def test_colsum(k):
    dy = _rand(777, 520, seed=1)
    out = torch.zeros(520, dtype=torch.float32, device="cuda")
    k.colsum_accumulate(dy.cuda(), out)
    _close(out, dy.float().sum(0), atol=1e-2, rtol=1e-3)


@pytest.mark.parametrize("d,hq,hkv", [(64, 4, 2), (128, 2, 2)])
def test_rope(k, d, hq, hkv):
    B, S = 2, 96
    qkv = _rand(B * S, (hq + 2 * hkv) * d, seed=1)
    cs = ref.rope_table(S, d, 10000.0)
    want = ref.rope(qkv.float(), cs, S, hq + hkv, d)
    got = k.rope_(qkv.cuda().clone(), cs.cuda(), S, hq + hkv, d)
    _close(got, want, atol=2e-2, rtol=1e-2)
    wantb = ref.rope(qkv.float(), cs, S, hq + hkv, d, backward=True)
    gotb = k.rope_(qkv.cuda().clone(), cs.cuda(), S, hq + hkv, d, backward=True)
    _close(gotb, wantb, atol=2e-2, rtol=1e-2)


def test_swiglu_and_act(k):
    T, F_ = 130, 1376
    gu, dout = _rand(T, 2 * F_, seed=1), _rand(T, F_, seed=2)
    gr = gu.float().requires_grad_(True)
    o = torch.nn.functional.silu(gr[:, :F_]) * gr[:, F_:]
    o.backward(dout.float())
    _close(k.swiglu_fwd(gu.cuda()), o.detach(), atol=2e-2, rtol=1e-2)
    _close(k.swiglu_bwd(gu.cuda(), dout.cuda()), gr.grad, atol=3e-2, rtol=2e-2)
    for kind, name in ((k.ACT_GELU_TANH, "gelu"), (k.ACT_RELU, "relu"), (k.ACT_GELU_ERF, "gelu_erf")):
        x = _rand(T, F_, seed=3)
        xr = x.float().requires_grad_(True)
        y = ref.activation(xr, name)
        y.backward(dout.float())
        _close(k.act_fwd(x.cuda(), kind), y.detach(), atol=2e-2, rtol=1e-2)
        _close(k.act_bwd(x.cuda(), dout.cuda(), kind), xr.grad, atol=3e-2, rtol=2e-2)


def test_embedding(k):
    V, H, S, B = 1000, 512, 16, 3
    table, pos = _rand(V, H, seed=1), _rand(S + 2, H, seed=2)
    ids = torch.randint(0, V, (B * S,), generator=torch.Generator().manual_seed(0))
    want = ref.embedding(ids, table.float(), pos.float(), S, 2)
    got = k.embedding_fwd(ids.cuda(), table.cuda(), pos.cuda(), S, 2)
    _close(got, want, atol=2e-2, rtol=1e-2)
    dout = _rand(B * S, H, seed=3)
    for gdt in (torch.float32, torch.bfloat16):
        dt = torch.zeros(V, H, dtype=gdt, device="cuda")
        dp = torch.zeros(S + 2, H, dtype=gdt, device="cuda")
        k.embedding_bwd(ids.cuda(), dout.cuda(), dt, dp, S, 2)
        wt = torch.zeros(V, H).index_add_(0, ids, dout.float())
        wp = torch.zeros(S + 2, H).index_add_(0, torch.arange(B * S) % S + 2, dout.float())
        _close(dt, wt, atol=5e-2, rtol=2e-2)
        _close(dp, wp, atol=5e-2, rtol=2e-2)


@pytest.mark.parametrize("T,V", [(9, 32000), (64, 50272), (4, 1001)])
def test_cross_entropy(k, T, V):
    logits = _rand(T, V, seed=1, scale=2.0)
    tg = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(1))
    lr = logits.float().requires_grad_(True)
    rows = torch.nn.functional.cross_entropy(lr, tg, reduction="none")
    (rows.sum() * 0.125).backward()
    d = torch.empty_like(logits, device="cuda")
    got = k.cross_entropy(logits.cuda(), tg.cuda(), 0.125, dlogits=d)
    _close(got, rows.detach(), atol=2e-3, rtol=1e-3)
    _close(d, lr.grad, atol=2e-3, rtol=2e-2)


def test_cross_entropy_ignored_rows(k):
    """Rows whose target is the ignore index (-100) give zero loss and a zero gradient row."""
    T, V = 64, 1000
    logits = _rand(T, V, seed=3, scale=2.0)
    tg = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(3))
    tg[::4] = -100
    lr = logits.float().requires_grad_(True)
    rows = torch.nn.functional.cross_entropy(lr, tg, reduction="none", ignore_index=-100)
    rows.sum().backward()
    d = torch.empty_like(logits, device="cuda")
    got = k.cross_entropy(logits.cuda(), tg.cuda(), 1.0, dlogits=d)
    _close(got, rows.detach(), atol=2e-3, rtol=1e-3)
    _close(d, lr.grad, atol=2e-3, rtol=2e-2)
    assert float(d[::4].float().abs().max()) == 0.0 and float(got[::4].abs().max()) == 0.0


@pytest.mark.parametrize("gdt", [torch.float32, torch.bfloat16])
def test_adam(k, gdt):
    n = 100_003
    g0 = torch.Generator().manual_seed(0)
    p = torch.randn(n, generator=g0)
    grads = [torch.randn(n, generator=g0).to(gdt) for _ in range(3)]
    pr = p.clone().requires_grad_(True)
    opt = torch.optim.Adam([pr], lr=1e-3, betas=(0.9, 0.999), eps=1e-8)
    pd, m, v = p.cuda(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    p16 = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    for step, g in enumerate(grads, 1):
        pr.grad = g.float() * 0.5
        opt.step()
        gd = g.cuda()
        k.adam_step(pd, m, v, gd, p16, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=step,
                    grad_scale=0.5, zero_grad=True)
        assert float(gd.float().abs().max()) == 0.0
    _close(pd, pr.detach(), atol=2e-6, rtol=1e-5)
    _close(p16, pr.detach(), atol=1e-2, rtol=1e-2)


ATTN_CASES = [
    (1, 300, 2, 1, 64, True, 0),
    (1, 640, 1, 1, 128, True, 200),
    # B, S, Hq, Hkv, D, causal, window
    (1, 128, 1, 1, 128, True, 0),
    (1, 128, 1, 1, 64, True, 0),
    (2, 256, 4, 2, 128, True, 0),
    (1, 384, 4, 1, 64, True, 0),
    (1, 200, 2, 2, 128, True, 0),
    (1, 512, 2, 1, 128, True, 192),
    (1, 256, 2, 2, 64, False, 0),
    (1, 1024, 2, 2, 128, True, 0),
]


# (version, flags)
FWD_VERSIONS = [(1, 0), (2, 0), (4, 0), (4, 1), (4, 2)]


@pytest.mark.parametrize("version,flags", FWD_VERSIONS)
@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal,window", ATTN_CASES)
def test_flash_fwd(k, B, S, Hq, Hkv, D, causal, window, version, flags):
    qkv = _rand(B * S, (Hq + 2 * Hkv) * D, seed=1)
    want = ref.attention(qkv.float(), B, S, Hq, Hkv, D, causal, window)
    out, lse = k.flash_fwd(qkv.cuda(), B, S, Hq, Hkv, D, causal, window, version=version, flags=flags)
    k.check_status()
    _close(out, want, atol=2e-2, rtol=2e-2)
    # log-sum-exp against the oracle's scores
    x = qkv.float().reshape(B, S, Hq + 2 * Hkv, D)
    q = x[:, :, :Hq].permute(0, 2, 1, 3)
    kk = x[:, :, Hq:Hq + Hkv].permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    s = (q @ kk.transpose(-1, -2)) / math.sqrt(D)
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    mask = torch.ones(S, S, dtype=torch.bool)
    if causal:
        mask &= j <= i
    if window:
        mask &= (i - j) < window
    want_lse = torch.logsumexp(s.masked_fill(~mask, float("-inf")), dim=-1)
    _close(lse, want_lse, atol=2e-2, rtol=1e-2)


def test_flash_default_versions_on_a_large_problem(k):
    """The size-based default picks the two-tile forward here (20 heads x 8 pairs of query tiles >= 148 CTAs);
    forward and backward defaults against the fp32 oracle, grouped-query heads, 2048 tokens."""
    B, S, Hq, Hkv, D = 1, 2048, 20, 4, 128
    assert k._auto_fwd_version(B, S, Hq) == 4 and k._auto_fwd_version(1, 1000, 8) == 1
    qkv = _rand(B * S, (Hq + 2 * Hkv) * D, seed=11)
    do = _rand(B * S, Hq * D, seed=12)
    q = qkv.float().requires_grad_(True)
    want_o = ref.attention(q, B, S, Hq, Hkv, D, True, 0)
    (want,) = torch.autograd.grad(want_o, q, do.float())
    out, lse = k.flash_fwd(qkv.cuda(), B, S, Hq, Hkv, D, True, 0)
    got = k.flash_bwd(do.cuda(), qkv.cuda(), out, lse, B, S, Hq, Hkv, D, True, 0)
    k.check_status()
    _close(out, want_o.detach(), atol=2e-2, rtol=2e-2)
    _close(got, want, atol=4e-2, rtol=3e-2)


BWD_VERSIONS = [1, 2, 3]


@pytest.mark.parametrize("version", BWD_VERSIONS)
@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal,window", ATTN_CASES)
def test_flash_bwd(k, B, S, Hq, Hkv, D, causal, window, version):
    qkv = _rand(B * S, (Hq + 2 * Hkv) * D, seed=1)
    do = _rand(B * S, Hq * D, seed=2)
    q = qkv.float().requires_grad_(True)
    want_o = ref.attention(q, B, S, Hq, Hkv, D, causal, window)
    (want,) = torch.autograd.grad(want_o, q, do.float())
    out, lse = k.flash_fwd(qkv.cuda(), B, S, Hq, Hkv, D, causal, window)
    for _ in range(2):  # second call checks that the scratch accumulator was left clean
        got = k.flash_bwd(do.cuda(), qkv.cuda(), out, lse, B, S, Hq, Hkv, D, causal, window, version=version)
    k.check_status()
    _close(got, want, atol=4e-2, rtol=3e-2)


def test_attention_traces_run(k):
    """The in-kernel phase traces terminate, leave the status word clean and record plausible clocks."""
    from zorse_b200.profiler import attn_trace

    for kern in ("fwd4", "bwd2"):
        attn_trace.main(["--kernel", kern, "--S", "1024", "--heads", "2", "--kv_heads", "2", "--ctas", "2"])
        k.check_status()


def test_a_wait_that_runs_out_reports_and_leaves_the_context_usable(k):
    """Failure detection on the device: a wait on a flag that nothing sets gives up after its (short)
    limit, the kernel returns, the host reads which wait it was, and the next launches work.  Nothing
    here faults, traps or spins without bound."""
    from zorse_b200.ops.sm100 import KernelError

    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    k.check_status()
    k.wait_flags(flags, 2, 0, 1, wait_seconds=0.05)        # flags[0..1] never reach epoch 1
    torch.cuda.synchronize()
    with pytest.raises(KernelError, match="status"):
        k.check_status()
    k.check_status()                                        # the word was cleared by the report
    flags[:2] = 1
    k.wait_flags(flags, 2, 0, 1, wait_seconds=0.05)        # satisfied at once
    k.check_status()
    x = torch.arange(8, device="cuda", dtype=torch.float32)
    assert float(x.sum().item()) == 28.0


@pytest.mark.skipif(not CANDIDATES, reason="ZORSE_TEST_CANDIDATES=1: first run on hardware pending")
@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(512, 768, 1024, True, True), (300, 520, 256, True, True),
                                              (512, 512, 512, False, False), (256, 1000, 384, False, True)])
def test_accumulate_prefetch_gemm_matches_the_default(k, M, N, K, a_mn, b_mn):
    """The accumulating GEMM that reads the old C tile ahead of the accumulators must give the default kernel's
    result bit for bit (same arithmetic, same order), ragged edges included, twice in a row."""
    g = torch.Generator(device="cuda").manual_seed(M + N)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).to(torch.bfloat16)
    c0 = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    want, got = c0.clone(), c0.clone()
    for _ in range(2):
        k.gemm(a, b, want, a_mn=a_mn, b_mn=b_mn, accumulate=True, kernel="2cta")
        k.gemm(a, b, got, a_mn=a_mn, b_mn=b_mn, accumulate=True, kernel="2cta_accpf")
    k.check_status()
    assert torch.equal(got, want)


def test_checking_build_gives_the_same_results_and_a_clean_status():
    """The debug build (-DZB_DEBUG_BOUNDS=1: kernels verify tile coordinates, shard offsets and flag indices and
    report through the status word) runs a GEMM with ragged edges and attention forward + backward in a child
    process and must agree with the fp32 oracle with no check tripped."""
    import subprocess
    import sys

    code = r'''
import math, torch
from zorse_b200.ops import sm100 as k
assert str(k.lib()._name).endswith("libzorse_sm100_dbg.so"), k.lib()._name
g = torch.Generator().manual_seed(3)
rnd = lambda *s: (torch.randn(*s, generator=g) * 0.5).to(torch.bfloat16)
a, b = rnd(300, 520), rnd(1320, 520)
out = torch.empty(300, 1320, dtype=torch.bfloat16, device="cuda")
k.gemm(a.cuda(), b.cuda(), out)
k.check_status()
want = a.float() @ b.float().t()
assert (out.float().cpu() - want).abs().max() < 0.15
B, S, Hq, Hkv, D = 1, 600, 4, 2, 128
qkv, do = rnd(B * S, (Hq + 2 * Hkv) * D).cuda(), rnd(B * S, Hq * D).cuda()
o1, l1 = k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, 0, version=1)
o4, l4 = k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, 0, version=4)
d1 = k.flash_bwd(do, qkv, o1, l1, B, S, Hq, Hkv, D, True, 0, version=1)
d3 = k.flash_bwd(do, qkv, o1, l1, B, S, Hq, Hkv, D, True, 0, version=3)
k.check_status()
assert (o1.float() - o4.float()).abs().max() < 3e-2 and (d1.float() - d3.float()).abs().max() < 6e-2
print("CHECKING_BUILD_OK")
'''
    env = dict(os.environ, ZORSE_DEBUG_BOUNDS="1")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=env,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "CHECKING_BUILD_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
