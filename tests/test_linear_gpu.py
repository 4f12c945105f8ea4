"""W8A8 linear on the GPU against the plain PyTorch reference of the same op."""
import pytest
import torch

from mojo_linuxperiments_b200.oracle import quant as Q

pytestmark = pytest.mark.gpu


def _mk_x(m, k, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((m, k), generator=g)
    mask = torch.rand((m, k), generator=g) < 1e-3
    x = torch.where(mask, x * 50, x)
    return x.to(torch.bfloat16).cuda()


def _mk_w(n, k, seed=1):
    g = torch.Generator(device="cpu").manual_seed(seed)
    wq = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).cuda()
    sw = (torch.rand((n,), generator=g) * 9e-3 + 1e-3).cuda()
    return wq, sw


@pytest.mark.parametrize("m,k", [(1, 128), (3, 512), (32, 4096), (257, 1792), (64, 14336)])
def test_act_quant_plain(m, k):
    from mojo_linuxperiments_b200.ops import linear as L
    x = _mk_x(m, k)
    q, s = L.act_quant(x)
    torch.cuda.synchronize()
    q_ref, s_ref = Q.rotate_quantize(x)
    assert torch.allclose(s, s_ref, rtol=1e-5, atol=0)
    d = (q.int() - q_ref.int()).abs()
    assert d.max().item() <= 1
    assert (d > 0).float().mean().item() < 2e-3


@pytest.mark.parametrize("mode", ["norm", "add_norm", "swiglu"])
def test_act_quant_fused_modes(mode):
    from mojo_linuxperiments_b200.ops import linear as L
    m, k = 37, 4096
    x = _mk_x(m, k, 3)
    gamma = (torch.rand(k) + 0.5).to(torch.bfloat16).cuda()
    if mode == "norm":
        q, s, xn = L.act_quant(x, mode=L.AQ_NORM, gamma=gamma, eps=1e-5, want_normed=True)
        ref = Q.rmsnorm(x, gamma, 1e-5)
        assert torch.allclose(xn.float(), ref, rtol=2e-2, atol=2e-2)
    elif mode == "add_norm":
        res = _mk_x(m, k, 4)
        res0 = res.clone()
        q, s = L.act_quant(x, mode=L.AQ_ADD_NORM, gamma=gamma, eps=1e-5, residual=res)
        h = (x.float() + res0.float()).to(torch.bfloat16)
        assert torch.equal(res, h)
        ref = Q.rmsnorm(h, gamma, 1e-5)
    else:
        gu = torch.cat([x, _mk_x(m, k, 5)], dim=1).contiguous()
        q, s = L.act_quant(gu, mode=L.AQ_SWIGLU)
        ref = Q.swiglu(gu)
    torch.cuda.synchronize()
    q_ref, s_ref = Q.quantize_rows(Q.rotate(ref))
    assert torch.allclose(s, s_ref, rtol=2e-3)
    deq = q.float() * s[:, None]
    deq_ref = q_ref.float() * s_ref[:, None]
    assert (deq - deq_ref).abs().max().item() <= 2.5 * s_ref.max().item()


GEMM_SHAPES = [
    (128, 128, 4096), (200, 128, 2048), (256, 128, 512), (65, 100, 640),      # narrow outputs: several 64-token tiles on the cluster kernel
    (16, 128, 128), (1, 128, 128), (1, 256, 512), (7, 384, 1024), (32, 4096, 4096), (32, 6144, 4096),
    (33, 1024, 512), (100, 4096, 1792), (128, 3584, 4096), (200, 1000, 768), (1024, 3584, 4096),
    (4096, 1792, 4096), (777, 16032, 1024),
]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("force_mode", [-1, 0, 1])
def test_w8a8_gemm_exact(m, n, k, force_mode):
    """Integer accumulation is exact, so the bf16 output may differ from the reference only by its rounding."""
    from mojo_linuxperiments_b200.ops import linear as L
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    if force_mode == 1 and m > 512:
        pytest.skip("stream-K is the small-M path")
    g = torch.Generator(device="cpu").manual_seed(m * 31 + n)
    xq = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).cuda()
    sx = (torch.rand((m,), generator=g) * 0.05 + 0.01).cuda()
    wq, sw = _mk_w(n, k)
    narrow = force_mode == -1 and n <= 128          # several 64-token tiles of the cluster kernel for narrow outputs
    y = L.w8a8_gemm(xq, sx, wq, sw, out_dtype=torch.float32, force_mode=force_mode, narrow=narrow)
    yb = L.w8a8_gemm(xq, sx, wq, sw, force_mode=force_mode, narrow=narrow)
    torch.cuda.synchronize()
    ws = default_workspace(xq.device)
    ws.check_status()
    assert int(ws.counters.abs().max().item()) == 0
    ref = Q.w8a8_linear(xq, sx, wq, sw)
    assert torch.allclose(y, ref, rtol=1e-5, atol=1e-5), (y - ref).abs().max().item()
    assert torch.allclose(yb.float(), ref, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (1, 6144, 4096), (16, 768, 4096), (17, 1000, 512), (32, 4096, 1792),
                                   (32, 4096, 512), (33, 3584, 4096), (64, 28672, 4096), (50, 4096, 14336), (3, 16032, 256)])
@pytest.mark.parametrize("splits", [0, 1, 2, 3, 4, 5, 6, 7, 8])
def test_w8a8_gemm_cluster_splitk(m, n, k, splits):
    """Decode kernel: split-K across a thread-block cluster, reduced through distributed shared memory."""
    from mojo_linuxperiments_b200.ops import linear as L
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    if splits and k // 128 < splits:
        pytest.skip("fewer k-blocks than splits is exercised by the auto choice only")
    g = torch.Generator(device="cpu").manual_seed(m * 7 + n + splits)
    xq = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).cuda()
    sx = (torch.rand((m,), generator=g) * 0.05 + 0.01).cuda()
    wq, sw = _mk_w(n, k)
    res = _mk_x(m, n, 11)
    y = L.w8a8_gemm(xq, sx, wq, sw, out_dtype=torch.float32, force_mode=2, force_splits=splits)
    yb = L.w8a8_gemm(xq, sx, wq, sw, residual=res, force_mode=2, force_splits=splits)
    torch.cuda.synchronize()
    default_workspace(xq.device).check_status()
    ref = Q.w8a8_linear(xq, sx, wq, sw)
    assert torch.allclose(y, ref, rtol=1e-5, atol=1e-5), (y - ref).abs().max().item()
    assert torch.allclose(yb.float(), ref + res.float(), rtol=1e-2, atol=2e-2)


def test_w8a8_gemm_residual_and_full_op():
    from mojo_linuxperiments_b200.ops import linear as L
    m, n, k = 48, 4096, 4096
    x = _mk_x(m, k)
    w = torch.randn((n, k), generator=torch.Generator().manual_seed(5)) * 0.02
    wq, sw = Q.quantize_weight(w.cuda())
    res = _mk_x(m, n, 9)
    q, s = L.act_quant(x)
    y = L.w8a8_gemm(q, s, wq, sw, residual=res)
    torch.cuda.synchronize()
    ref_same_q = Q.w8a8_linear(q, s, wq, sw, residual=res)
    assert torch.allclose(y.float(), ref_same_q, rtol=1e-2, atol=2e-2)
    # looser: against the unquantised product
    exact = x.float() @ w.cuda().t() + res.float()
    rel = (y.float() - exact).norm() / exact.norm()
    assert rel.item() < 0.05


@pytest.mark.parametrize("mode", ["plain", "norm", "add_norm", "swiglu"])
@pytest.mark.parametrize("m,n,k", [(1, 768, 4096), (32, 6144, 4096), (17, 4096, 1792), (64, 1024, 512), (32, 4096, 14336)])
def test_fused_linear_runs_its_own_activation_prologue(mode, m, n, k):
    """One launch from bf16 rows to the linear's output: the quantiser CTAs inside the GEMM launch must produce what the
    stand-alone prologue + GEMM produce (same int8 rows up to rare +-1 ties, so the outputs agree closely), update the
    residual exactly, and keep doing so when the launch is replayed from a CUDA graph."""
    from mojo_linuxperiments_b200.ops import linear as L
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    ws = default_workspace(torch.device("cuda", 0))
    wq, sw = _mk_w(n, k)
    gamma = (torch.rand(k) + 0.5).to(torch.bfloat16).cuda()
    x = _mk_x(m, 2 * k if mode == "swiglu" else k, 21)
    res = _mk_x(m, k, 22)

    def unfused():
        if mode == "plain":
            q, s = L.act_quant(x)
        elif mode == "norm":
            q, s = L.act_quant(x, mode=L.AQ_NORM, gamma=gamma, eps=1e-5)
        elif mode == "add_norm":
            r = res.clone()
            q, s = L.act_quant(x, mode=L.AQ_ADD_NORM, gamma=gamma, eps=1e-5, residual=r)
            return L.w8a8_gemm(q, s, wq, sw, force_mode=2), r
        else:
            q, s = L.act_quant(x, mode=L.AQ_SWIGLU)
        return L.w8a8_gemm(q, s, wq, sw, force_mode=2), None

    def fused(r):
        md = {"plain": L.QR_PLAIN, "norm": L.QR_NORM, "add_norm": L.QR_ADD_NORM, "swiglu": L.QR_SWIGLU}[mode]
        return L.fused_linear(x, wq, sw, mode=md, gamma=gamma if mode in ("norm", "add_norm") else None, eps=1e-5,
                              residual=r if mode == "add_norm" else None)

    ref, ref_res = unfused()
    r1 = res.clone()
    y1 = fused(r1)
    ws.next_step()
    r2 = res.clone()
    y2 = fused(r2)
    torch.cuda.synchronize()
    ws.check_status()
    tol = 2e-2 * ref.float().abs().max().item()
    assert torch.allclose(y1.float(), ref.float(), rtol=2e-2, atol=tol), (y1.float() - ref.float()).abs().max().item()
    assert torch.equal(y1, y2)
    if mode == "add_norm":
        assert torch.equal(r1, ref_res) and torch.equal(r2, ref_res)
    # replayed from a graph: the step word moves between replays, the row flags are told apart by it
    rg = res.clone()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            yg = fused(rg)
            yg2 = fused(rg) if mode != "add_norm" else yg
            ws.next_step()
    for _ in range(3):
        rg.copy_(res)
        g.replay()
    torch.cuda.synchronize()
    ws.check_status()
    assert torch.equal(yg, y1) and torch.equal(yg2, y1)


@pytest.mark.parametrize("mode", ["plain", "norm", "add_norm", "swiglu"])
@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("n,k", [(768, 4096), (6144, 4096), (4096, 1792), (28672, 4096), (4096, 14336), (512, 128), (1000, 640)])
def test_fused_linear_inline_prologue_for_a_few_tokens(mode, m, n, k):
    """Up to four tokens the GEMM CTAs quantise their own operand (row statistics exchanged inside the split-K cluster).
    The result must match stand-alone prologue + GEMM (the rotation runs before the norm's 1/rms is applied, so single
    int8 values may differ by one step), the residual sum goes to the second buffer bit-exactly and the input residual
    stays untouched; shapes whose K slice does not fit a warp's registers fall back to quantiser CTAs and must agree too."""
    from mojo_linuxperiments_b200.ops import linear as L
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    ws = default_workspace(torch.device("cuda", 0))
    wq, sw = _mk_w(n, k)
    gamma = (torch.rand(k) + 0.5).to(torch.bfloat16).cuda()
    x = _mk_x(m, 2 * k if mode == "swiglu" else k, 31)
    res = _mk_x(m, k, 32)
    md = {"plain": L.QR_PLAIN, "norm": L.QR_NORM, "add_norm": L.QR_ADD_NORM, "swiglu": L.QR_SWIGLU}[mode]
    aq = {"plain": L.AQ_PLAIN, "norm": L.AQ_NORM, "add_norm": L.AQ_ADD_NORM, "swiglu": L.AQ_SWIGLU}[mode]
    r_ref = res.clone()
    q, s = L.act_quant(x, mode=aq, gamma=gamma if mode in ("norm", "add_norm") else None, eps=1e-5,
                       residual=r_ref if mode == "add_norm" else None)
    ref = L.w8a8_gemm(q, s, wq, sw, force_mode=2)
    r_in, r_out = res.clone(), torch.full_like(res, 7.0)

    def fused():
        return L.fused_linear(x, wq, sw, mode=md, gamma=gamma if mode in ("norm", "add_norm") else None, eps=1e-5,
                              residual=r_in if mode == "add_norm" else None, residual_out=r_out if mode == "add_norm" else None,
                              inline=True)

    y1 = fused()
    ws.next_step()
    y2 = fused()
    torch.cuda.synchronize()
    ws.check_status()
    rel = ((y1.float() - ref.float()).norm() / ref.float().norm()).item()
    assert rel < 1e-2, rel
    assert torch.equal(y1, y2)
    if mode == "add_norm":
        assert torch.equal(r_out, r_ref) and torch.equal(r_in, res)
    g = torch.cuda.CUDAGraph()
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        with torch.cuda.graph(g, stream=st):
            yg = fused()
            ws.next_step()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ws.check_status()
    assert torch.equal(yg, y1)
