"""The reference's own unfused GPU operators (bst_sgemm_nt -> BlocksparseMaskedSoftmax -> bst_sgemm_xn, compiled for
sm_100a from the reference header into oracle/_ref/libsfb_ref_gpu.so) run on this GPU beside the product path and the
CPU oracle, on the same seeded inputs.  The reference implements these for block size 32 with fp32 activations and
bf16 scores / probabilities, so the comparisons carry the 16-bit bar (2e-2 relative); the score tiles, one bf16
rounding of an fp32 dot product on both sides, must agree to one bf16 unit in the last place.
The reference's fused kernels wait on global flags without a bound and are never launched."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def trio(oracle):
    if oracle.ref_gpu() is None:
        pytest.skip("oracle/_ref/libsfb_ref_gpu.so was not built (needs the reference tree at build time)")
    return oracle


def _qkv(oracle, shape, seed):
    return [torch.from_numpy(oracle.fill_normal(shape, seed + i)).cuda() for i in range(3)]


def _within(a, b, bound, what):
    """Element-wise |a - b| <= bound, with the worst offender in the message."""
    diff = (a - b).abs()
    bad = diff > bound
    n = int(bad.sum())
    if n:
        i = int((diff - bound).argmax())
        raise AssertionError("%s: %d of %d elements out of bound; worst a=%r b=%r bound=%r" % (
            what, n, diff.numel(), float(a.flatten()[i]), float(b.flatten()[i]),
            float(bound.flatten()[i]) if torch.is_tensor(bound) else bound))


CASES = [
    # name, oracle layout kind + args, device layout kind + args, heads in the LUT, B, H, L
    ("fixed_cfg", "fixed", dict(stride=4), ("LAYOUT_FIXED", dict(p0=4)), 4, 1, 4, 512),
    ("stride", "stride", dict(band=4, every=8), ("LAYOUT_STRIDE", dict(p0=4, p1=8)), 1, 2, 4, 1024),
    ("local", "local", dict(left=2, right=2), ("LAYOUT_LOCAL", dict(p0=2, p1=2)), 1, 2, 3, 2048),
    ("full", "full", dict(), ("LAYOUT_FULL", dict()), 1, 1, 2, 256),
]


@pytest.mark.parametrize("name,kind,kw,dev,lut_heads,B,H,L", CASES)
def test_reference_gpu_operators_against_product_and_oracle(sfb, trio, name, kind, kw, dev, lut_heads, B, H, L):
    O = trio
    d, bs = 64, 32
    nb = L // bs
    scale = float(np.float32(1.0 / np.sqrt(d)))
    layout = O.layout(kind, lut_heads, nb, **kw)
    luts = O.lut_build(layout)
    q, k, v = _qkv(O, (B, L, H, d), 900)
    ref = O.RefGpuAttention(layout)

    lay = sfb.BlockLayout.generate(getattr(sfb, dev[0]), lut_heads, nb, bs, **dev[1])
    assert lay.blocks == ref.blocks and lay.nn_max == ref.nn_max
    assert torch.equal(lay.nt_lut, ref.nt) and torch.equal(lay.nn_lut, ref.nn)

    # --- SDDMM: both round an fp32 dot product of the same operands to bf16 once
    ref.alloc(q)
    ref.launch(q, k, v, scale)
    torch.cuda.synchronize()
    s_ref = ref.s.float()
    s_ours = sfb.bst_sgemm_nt(q, k, lay, out_dtype=torch.bfloat16).float()
    # one bf16 unit in the last place; the floor covers fp32 summation order on scores that cancel to nearly zero
    ulp = torch.maximum(s_ref.abs(), s_ours.abs()) * 2.0 ** -7 + 1e-4
    _within(s_ref, s_ours, ulp, "scores, reference GPU against product")
    assert float((s_ref == s_ours).float().mean()) > 0.98
    cpu = O.attention(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), luts, bs, np.float32(scale), round_s_bf16=True)
    s_cpu = torch.from_numpy(cpu["s"]).cuda()
    _within(s_ref, s_cpu, ulp, "scores, reference GPU against CPU oracle")

    # --- softmax on the SAME score tensor (the reference's), bf16 out
    p_ref = ref.p.float()
    p_ours = sfb.masked_softmax(ref.s, lay, scale, out_dtype=torch.bfloat16).float()
    tol = 2e-2 * torch.maximum(p_ref, p_ours) + 1e-6
    _within(p_ref, p_ours, tol, "probabilities")
    # --- SpMM on the SAME probabilities (the reference's)
    o_ref = ref.o
    o_ours = sfb.bst_sgemm_xn(ref.p, v, lay)
    assert float((o_ref - o_ours).abs().max()) <= 1e-4 * float(o_ref.abs().max()) + 1e-5

    # --- end to end: the product's fused fp32 kernel and the oracle against the reference's three launches
    o_fused = sfb.fused_attention(q, k, v, lay, scale)
    o_cpu = torch.from_numpy(cpu["o"]).cuda()
    bar = 2e-2 * float(o_ref.abs().max())
    assert float((o_ref - o_fused).abs().max()) <= bar
    assert float((o_ref - o_cpu).abs().max()) <= bar
    assert sfb.device_status() == 0


def test_reference_gpu_softmax_float_rows_sum_to_one(sfb, trio):
    """The <float,float2> instantiation the fixed-pattern test program uses (fixed_fusion_test.cu:435)."""
    O = trio
    B, H, L, d, bs = 1, 4, 512, 64, 32
    nb = L // bs
    scale = float(np.float32(1.0 / np.sqrt(d)))
    layout = O.layout("fixed", 4, nb, stride=4)
    q, k, v = _qkv(O, (B, L, H, d), 910)
    ref = O.RefGpuAttention(layout)
    ref.alloc(q, p_float=True)
    ref.launch(q, k, v, scale)
    torch.cuda.synchronize()
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_FIXED, 4, nb, bs, p0=4)
    p_ours = sfb.masked_softmax(ref.s, lay, scale, out_dtype=torch.float32)
    p_ref = ref.p
    # the reference rounds every exponential to bf16 before it normalises (blocksparse.h:605): 2^-8 relative
    _within(p_ref, p_ours, 2.0 ** -7 * torch.maximum(p_ref, p_ours) + 1e-7, "fp32 probabilities")
    # row sums of the product's probabilities, gathered per query row through the nt LUT
    nt = lay.nt_lut.cpu().numpy()
    sums = np.zeros((B, H, L), np.float64)
    rs = p_ours.double().sum(-1).cpu().numpy()                    # [B,H,blocks,bs]
    for h in range(H):
        for kk in range(lay.blocks):
            i = int(nt[h, kk, 0])
            sums[:, h, i * bs:(i + 1) * bs] += rs[:, h, kk]
    assert np.abs(sums - 1.0).max() <= 1e-3


def test_same_mask_on_blocks_of_64_and_32(sfb, trio):
    """bench.py's reference arm runs the reference on the bench layout split into 32x32 blocks (the only size
    its matmuls implement).  The product's tensor-core kernel on the 64x64 layout must give the same attention."""
    O = trio
    B, H, L, d = 2, 4, 2048, 64
    scale = float(np.float32(1.0 / np.sqrt(d)))
    lay64_np = O.layout("stride", 1, L // 64, band=4, every=8)
    lay32_np = O.split_layout(lay64_np)
    assert int(lay32_np.sum()) == 4 * int(lay64_np.sum())
    q, k, v = _qkv(O, (B, L, H, d), 920)
    ref = O.RefGpuAttention(lay32_np)
    ref.alloc(q)
    ref.launch(q, k, v, scale)
    torch.cuda.synchronize()
    lay64 = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, L // 64, 64, p0=4, p1=8)
    for dt in (torch.float16, torch.bfloat16):
        o = sfb.fused_attention(q.to(dt), k.to(dt), v.to(dt), lay64, scale).float()
        assert float((o - ref.o).abs().max()) <= 2e-2 * float(ref.o.abs().max())
    assert sfb.device_status() == 0


@pytest.mark.parametrize("kind,dev,nb", [("stride", ("LAYOUT_STRIDE", dict(p0=4, p1=8)), 32),
                                          ("local", ("LAYOUT_LOCAL", dict(p0=8, p1=8)), 48),
                                          ("full", ("LAYOUT_FULL", dict()), 8)])
def test_reference_gpu_softmax_at_block_64(sfb, trio, kind, dev, nb):
    """The reference's softmax is also implemented for 64x64 blocks (its matmuls are not): on the block size of the
    tensor-core kernels the product's stand-alone softmax must agree with it on the same bf16 scores."""
    import ctypes as C
    O = trio
    B, H, d, bs = 2, 4, 64, 64
    L = nb * bs
    scale = float(np.float32(1.0 / np.sqrt(d)))
    lay = sfb.BlockLayout.generate(getattr(sfb, dev[0]), 1, nb, bs, **dev[1])
    q, k, _ = _qkv(O, (B, L, H, d), 930)
    s = sfb.bst_sgemm_nt(q.to(torch.bfloat16), k.to(torch.bfloat16), lay, out_dtype=torch.bfloat16)
    p_ref = torch.empty_like(s)
    u, vp = C.c_uint32, lambda t: C.c_void_p(t.data_ptr())
    rc = O.ref_gpu().ref_gpu_masked_softmax(C.c_void_p(torch.cuda.current_stream().cuda_stream), vp(lay.nn_lut), None, vp(s),
                                            vp(p_ref), C.c_int(0), u(bs), u(lay.blocks), u(B), u(H), u(nb), u(1),
                                            u(lay.nn_lut_dim), u(lay.nn_max), u(1), C.c_float(scale))
    assert rc == 0, rc
    torch.cuda.synchronize()
    p_ours = sfb.masked_softmax(s, lay, scale, out_dtype=torch.bfloat16).float()
    p_ref = p_ref.float()
    _within(p_ref, p_ours, 2e-2 * torch.maximum(p_ref, p_ours) + 1e-6, "probabilities at block 64")
    assert sfb.device_status() == 0


@pytest.mark.parametrize("kind,kw,dev,lut_heads,B,H,L", [
    ("stride", dict(band=4, every=8), ("LAYOUT_STRIDE", dict(p0=4, p1=8)), 1, 2, 4, 1024),
    ("fixed", dict(stride=4), ("LAYOUT_FIXED", dict(p0=4)), 4, 1, 4, 512),
    ("local", dict(left=2, right=1), ("LAYOUT_LOCAL", dict(p0=2, p1=1)), 1, 1, 3, 1024),
])
def test_reference_gpu_backward_operators(sfb, trio, kind, kw, dev, lut_heads, B, H, L):
    """The reference's backward call sequence on this GPU (transformer_attention_optimize.cu:924-964: dV = P^T dO with
    TN_OP, dP = dO V^T, dS = softmax gradient, dK = dS^T Q, dQ = dS K) beside the product's, each operator fed with the
    reference's own inputs; block size 32, fp32 activations, bf16 block tensors."""
    import ctypes as C
    O = trio
    d, bs = 64, 32
    nb = L // bs
    scale = float(np.float32(1.0 / np.sqrt(d)))
    layout = O.layout(kind, lut_heads, nb, **kw)
    q, k, v = _qkv(O, (B, L, H, d), 940)
    do = torch.from_numpy(O.fill_normal((B, L, H, d), 944)).cuda()
    ref = O.RefGpuAttention(layout)
    ref.alloc(q)
    ref.launch(q, k, v, scale)
    lay = sfb.BlockLayout.generate(getattr(sfb, dev[0]), lut_heads, nb, bs, **dev[1])
    tn = O.lut_build_tn(layout)
    assert np.array_equal(lay.tn_lut.cpu().numpy().view(np.uint32), tn["tn"]) and lay.tn_max == tn["tn_max"]
    G = O.ref_gpu()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    u, vp = C.c_uint32, lambda t: C.c_void_p(t.data_ptr())
    p = ref.p                                                           # bf16 probabilities of the reference's forward

    def ref_tn(a, b):
        c = torch.empty_like(b)
        rc = G.ref_gpu_bst_sgemm_tn(st, vp(lay.tn_lut), vp(a), vp(b), vp(c), u(bs), u(lay.blocks), u(B), u(nb), u(nb), u(H), u(d),
                                    u(lut_heads), u(lay.blocks + nb), u(lay.tn_max))
        assert rc == 0, rc
        return c

    def close32(a, b, what):
        assert float((a - b).abs().max()) <= 1e-4 * float(a.abs().max()) + 1e-5, what

    # dV = P^T dO
    close32(ref_tn(p, do), sfb.bst_sgemm_tn(p, do, lay), "dV")
    # dP = dO V^T, rounded to bf16 once on both sides
    dp_ref = torch.empty_like(ref.s)
    rc = G.ref_gpu_bst_sgemm_nt(st, vp(ref.nt), vp(do), vp(v), vp(dp_ref), u(bs), u(lay.blocks), u(B), u(nb), u(nb), u(H), u(d),
                                u(lut_heads), u(lay.blocks))
    assert rc == 0, rc
    dp_ours = sfb.bst_sgemm_nt(do, v, lay, out_dtype=torch.bfloat16)
    a, b_ = dp_ref.float(), dp_ours.float()
    _within(a, b_, torch.maximum(a.abs(), b_.abs()) * 2.0 ** -7 + 1e-4, "dP")
    # dS from the reference's dP and P
    ds_ref = torch.empty_like(p)
    rc = G.ref_gpu_masked_softmax_grad(st, vp(ref.nn), vp(dp_ref), vp(p), vp(ds_ref), u(bs), u(lay.blocks), u(B), u(H), u(nb),
                                       u(lut_heads), u(lay.blocks + nb), u(lay.nn_max), C.c_float(scale))
    assert rc == 0, rc
    ds_ours = sfb.masked_softmax_grad(dp_ref, p, lay, scale)
    a, b_ = ds_ref.float(), ds_ours.float()
    _within(a, b_, torch.maximum(a.abs(), b_.abs()) * 2.0 ** -7 + 1e-5 * float(a.abs().max()) + 1e-7, "dS")
    # dK = dS^T Q and dQ = dS K from the reference's dS
    close32(ref_tn(ds_ref, q), sfb.bst_sgemm_tn(ds_ref, q, lay), "dK")
    dq_ref = torch.empty_like(q)
    rc = G.ref_gpu_bst_sgemm_nn(st, vp(ref.nn), vp(ds_ref), vp(k), vp(dq_ref), u(bs), u(lay.blocks), u(B), u(nb), u(nb), u(H), u(d),
                                u(lut_heads), u(lay.blocks + nb), u(lay.nn_max))
    assert rc == 0, rc
    close32(dq_ref, sfb.bst_sgemm_xn(ds_ref, k, lay), "dQ")
    torch.cuda.synchronize()
    assert sfb.device_status() == 0


def test_reference_gpu_softmax_grad_at_block_64(sfb, trio):
    import ctypes as C
    O = trio
    B, H, nb, bs = 2, 4, 32, 64
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_STRIDE, 1, nb, bs, p0=4, p1=8)
    g = torch.Generator(device="cuda").manual_seed(950)
    y = torch.rand(B, H, lay.blocks, bs, bs, device="cuda", generator=g).mul_(0.01).to(torch.bfloat16)
    dy = torch.randn(B, H, lay.blocks, bs, bs, device="cuda", generator=g).to(torch.bfloat16)
    dx_ref = torch.empty_like(y)
    u, vp = C.c_uint32, lambda t: C.c_void_p(t.data_ptr())
    rc = O.ref_gpu().ref_gpu_masked_softmax_grad(C.c_void_p(torch.cuda.current_stream().cuda_stream), vp(lay.nn_lut), vp(dy), vp(y),
                                                 vp(dx_ref), u(bs), u(lay.blocks), u(B), u(H), u(nb), u(1), u(lay.nn_lut_dim),
                                                 u(lay.nn_max), C.c_float(0.125))
    assert rc == 0, rc
    torch.cuda.synchronize()
    a, b_ = dx_ref.float(), sfb.masked_softmax_grad(dy, y, lay, 0.125).float()
    _within(a, b_, torch.maximum(a.abs(), b_.abs()) * 2.0 ** -7 + 1e-5 * float(a.abs().max()) + 1e-7, "dS at block 64")
