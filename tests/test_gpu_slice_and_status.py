"""Head slices of wider tensors (what a rank of a multi-GPU run computes), the device status word, and a second
device in one process -- all through the C ABI on the GPU."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,bs,d", [("bf16", 64, 64), ("f16", 64, 64), ("f32", 32, 64)])
@pytest.mark.parametrize("b0,b1,h0,h1", [(0, 1, 2, 5), (1, 3, 0, 6), (2, 3, 5, 6)])
def test_head_slice_equals_the_unsliced_call(sfb, dtype, bs, d, b0, b1, h0, h1):
    """sfb_fused_attention_slice on q[b0:b1, :, h0:h1] of [B, L, H, d] tensors, output written in place into the same
    slice of a full-size o, equals sfb_fused_attention on the whole tensors, bit for bit (tensor cores and CUDA cores)."""
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    B, H, L = 3, 6, 512
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, L // bs, bs, p0=3, p1=4)
    gen = torch.Generator(device="cuda").manual_seed(5)
    q, k, v = (torch.randn(B, L, H, d, device="cuda", generator=gen).to(tdt) for _ in range(3))
    want = sfb.fused_attention(q, k, v, lay, 0.125)
    o = torch.full_like(q, 7.0)
    sfb.fused_attention_slice(q[b0:b1, :, h0:h1], k[b0:b1, :, h0:h1], v[b0:b1, :, h0:h1], lay, 0.125, out=o[b0:b1, :, h0:h1])
    assert sfb.device_status() == 0
    assert torch.equal(o[b0:b1, :, h0:h1], want[b0:b1, :, h0:h1])
    # nothing outside the slice was touched
    keep = torch.ones(B, 1, H, 1, dtype=torch.bool, device="cuda")
    keep[b0:b1, :, h0:h1] = False
    assert bool(((o == 7.0) | ~keep).all())
    # a packed output (its own pitch) gives the same numbers
    packed = sfb.fused_attention_slice(q[b0:b1, :, h0:h1], k[b0:b1, :, h0:h1], v[b0:b1, :, h0:h1], lay, 0.125)
    assert packed.is_contiguous() and torch.equal(packed, want[b0:b1, :, h0:h1])


def test_slice_rejects_a_pitch_below_the_slice_width(sfb):
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_FULL, 1, 2, 64)
    q = torch.zeros(1, 128, 2, 64, device="cuda", dtype=torch.bfloat16)
    rc = sfb.lib.sfb_fused_attention_slice(None, C.c_void_p(lay.nn_lut.data_ptr()), C.c_void_p(q.data_ptr()), C.c_void_p(q.data_ptr()),
                                           C.c_void_p(q.data_ptr()), C.c_void_p(q.data_ptr()), None, sfb.BF16, 64, lay.blocks, 1, 2, 2, 64,
                                           1, lay.blocks, 1, 0.125, lay.nn_max, 64, 0)
    assert rc != 0 and b"pitch" in sfb.lib.sfb_last_error()


def test_status_word_reports_a_row_pair_that_is_too_long(sfb, oracle):
    """A caller that promises short rows (max_lut) but hands over a layout whose first row pair touches more key blocks
    than the tensor-core kernel's list holds: the kernel records code 9, writes that pair's rows as zeros, computes every
    other row, nothing hangs or faults, and after sfb_device_status_clear the next call is clean."""
    nb, d = 300, 64
    L = nb * 64
    layout = np.zeros((1, nb, nb), np.uint8)
    layout[0, 0, :] = 1
    layout[0, 1, :] = 1
    for i in range(2, nb):
        layout[0, i, i] = 1
    lay = sfb.BlockLayout(torch.from_numpy(layout).cuda(), 64)
    assert lay.nn_max == nb
    gen = torch.Generator(device="cuda").manual_seed(9)
    q, k, v = (torch.randn(1, L, 1, d, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(3))
    o = torch.full_like(q, 3.0)
    sfb.device_status_clear()
    p = lambda t: C.c_void_p(t.data_ptr())
    rc = sfb.lib.sfb_fused_attention(C.c_void_p(torch.cuda.current_stream().cuda_stream), p(lay.nn_lut), p(q), p(k), p(v), p(o), None,
                                     sfb.BF16, 64, lay.blocks, 1, nb, 1, d, 1, lay.blocks, 1, 0.125, 4)   # max_lut = 4 is the lie
    assert rc == 0
    status = sfb.device_status()
    assert status >> 24 == 9
    assert float(o[:, :128].abs().max()) == 0.0
    # every other block-row keeps its diagonal block only: attention inside 64-token windows
    rows = slice(128, L)
    win = lambda t: t[0, rows, 0].float().cpu().numpy().reshape(nb - 2, 64, 1, d)
    one = oracle.lut_build(oracle.layout("full", 1, 1))
    ref = oracle.attention(win(q), win(k), win(v), one, 64, np.float32(0.125), want=("o",))["o"]
    got = win(o)
    assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max()
    sfb.device_status_clear()
    assert sfb.device_status() == 0
    # the honest call (max_lut as built) takes the CUDA-core kernel for this layout and is clean
    o2 = sfb.fused_attention(q, k, v, lay, 0.125)
    assert sfb.device_status() == 0
    assert np.abs(win(o2) - ref).max() <= 2e-2 * np.abs(ref).max()
    assert float(o2[:, :128].abs().max()) > 0.0


def test_second_device_first(sfb, oracle):
    """A process whose first calls go to device 1: the kernels' launch set-up (shared-memory sizes, SM count) is kept per
    device, not per process."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with torch.cuda.device(1):
        lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, 8, 64, p0=4, p1=8, device="cuda:1")
        gen = torch.Generator(device="cuda:1").manual_seed(3)
        q, k, v = (torch.randn(2, 512, 2, 64, device="cuda:1", generator=gen).to(torch.bfloat16) for _ in range(3))
        o1 = sfb.fused_attention(q, k, v, lay, 0.125)
        x = torch.randn(256, 128, device="cuda:1", generator=gen).to(torch.bfloat16)
        w = torch.randn(128, 64, device="cuda:1", generator=gen).to(torch.bfloat16)
        y1 = sfb.linear(x, w)
        torch.cuda.synchronize()
    lay0 = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, 8, 64, p0=4, p1=8)
    o0 = sfb.fused_attention(q.to("cuda:0"), k.to("cuda:0"), v.to("cuda:0"), lay0, 0.125)
    y0 = sfb.linear(x.to("cuda:0"), w.to("cuda:0"))
    assert torch.equal(o0.cpu(), o1.cpu()) and torch.equal(y0.cpu(), y1.cpu())


def test_operands_the_tma_cannot_address_fall_back(sfb):
    """A score tensor that is 16-byte but not 32-byte aligned (and operands at an odd element) cannot go through the TMA
    kernels; the same call then runs on the CUDA cores instead of being rejected, with the same result up to rounding."""
    B, H, L, d = 1, 2, 512, 64
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, L // 64, 64, p0=3, p1=4)
    gen = torch.Generator(device="cuda").manual_seed(17)
    q, k, v = (torch.randn(B, L, H, d, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(3))
    s_ref = sfb.bst_sgemm_nt(q, k, lay, torch.bfloat16)
    n = s_ref.numel()
    buf = torch.empty(n + 8, dtype=torch.bfloat16, device="cuda")
    s_off = buf[8:].view_as(s_ref)                       # 16 bytes past a 256-byte boundary
    assert s_off.data_ptr() % 32 == 16
    p = lambda t: C.c_void_p(t.data_ptr())
    rc = sfb.lib.sfb_bst_sgemm_nt(C.c_void_p(torch.cuda.current_stream().cuda_stream), p(lay.nt_lut), p(q), p(k), p(s_off), sfb.BF16, sfb.BF16,
                                  64, lay.blocks, B, lay.nb, lay.nb, H, d, 1, lay.blocks)
    assert rc == 0, sfb.lib.sfb_last_error()
    assert float((s_off.float() - s_ref.float()).abs().max()) <= 2.0 ** -7 * float(s_ref.float().abs().max())
    # fused attention with q two bytes off: CUDA cores, same numbers at the 16-bit bar
    qb = torch.empty(q.numel() + 8, dtype=torch.bfloat16, device="cuda")
    q_off = qb[1:1 + q.numel()].view_as(q)
    q_off.copy_(q)
    want = sfb.fused_attention(q, k, v, lay, 0.125).float()
    got = sfb.fused_attention(q_off, k, v, lay, 0.125).float()
    assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bias_gelu_in_place(sfb, dtype):
    gen = torch.Generator(device="cuda").manual_seed(23)
    x = torch.randn(300, 256, device="cuda", generator=gen).to(dtype)
    bias = torch.randn(256, device="cuda", generator=gen)
    want = sfb.bias_gelu(x, bias)
    y = x.clone()
    sfb.bias_gelu(y, bias, out=y)
    assert torch.equal(y, want)


@pytest.mark.parametrize("dtype,hidden", [(torch.float32, 256), (torch.bfloat16, 768), (torch.float16, 1024)])
@pytest.mark.parametrize("target", ["x", "resid"])
def test_layernorm_in_place(sfb, dtype, hidden, target):
    """out may be x or resid themselves: a row is read completely before the warp that owns it writes it."""
    gen = torch.Generator(device="cuda").manual_seed(29)
    m = 5000          # more rows than resident warps: every warp also prefetches rows it writes later
    x, resid = (torch.randn(m, hidden, device="cuda", generator=gen).to(dtype) for _ in range(2))
    bias, gain, beta = (torch.randn(hidden, device="cuda", generator=gen) for _ in range(3))
    want, _, mean, rstd = sfb.bias_residual_layernorm(x, bias, resid, gain, beta)
    xs, rs = x.clone(), resid.clone()
    dst = xs if target == "x" else rs
    got, _, mean2, rstd2 = sfb.bias_residual_layernorm(xs, bias, rs, gain, beta, out=dst)
    assert got.data_ptr() == dst.data_ptr()
    assert torch.equal(got, want) and torch.equal(mean, mean2) and torch.equal(rstd, rstd2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hidden", [264, 520, 768, 1000, 1024, 1544, 2048])
@pytest.mark.parametrize("m,with_resid", [(1, True), (5, False), (1001, True), (20000, True)])
def test_layernorm_few_and_many_rows(sfb, dtype, hidden, m, with_resid):
    """Launches of few rows take the kernel with two warps per row, larger ones the persistent one-warp-per-row kernel;
    row lengths that do not fill the last 16-byte chunk of a lane, one row, and a row count that is no multiple of the
    rows per CTA.  Against a float64 LayerNorm of the same inputs (E[x^2] - mean^2, eps 1e-5 inside the root)."""
    gen = torch.Generator(device="cuda").manual_seed(hidden + m)
    x = torch.randn(m, hidden, device="cuda", generator=gen).to(dtype)
    resid = torch.randn(m, hidden, device="cuda", generator=gen).to(dtype) if with_resid else None
    bias, gain, beta = (torch.randn(hidden, device="cuda", generator=gen) for _ in range(3))
    out, summed, mean, rstd = sfb.bias_residual_layernorm(x, bias, resid, gain, beta, want_sum=True)
    t = x.double() + bias.double()
    if with_resid:
        t = t + resid.double()
    mu = t.mean(-1, keepdim=True)
    var = (t * t).mean(-1, keepdim=True) - mu * mu
    want = (t - mu) / torch.sqrt(var.clamp_min(0) + 1e-5) * gain.double() + beta.double()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((out.double() - want).abs().max()) <= tol * float(want.abs().max())
    assert float((summed.double() - t).abs().max()) <= (1e-6 if dtype == torch.float32 else 2e-2) * float(t.abs().max())
    assert float((mean.double() - mu.squeeze(-1)).abs().max()) <= 1e-5
    assert float((rstd.double() * torch.sqrt(var.clamp_min(0) + 1e-5).squeeze(-1) - 1).abs().max()) <= 1e-4

