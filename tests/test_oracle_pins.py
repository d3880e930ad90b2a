"""Pins the CPU oracle to the reference: (1) the LUT / mask arrays that the reference's own
test programs upload (tests/golden/ref_uploads.npz, made by tests/golden/make_golden.py),
(2) outputs of the reference's own CPU operators (tests/golden/ref_cpu_attention.npz), and
(3) the all-ones known answer of the reference test programs (fixed_fusion_test.cu:263-268,
test.cu:382-386: every score equals d, every probability 1/#kept)."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _layout_from_nt(nt, nb):
    lay = np.zeros((1, nb, nb), np.uint8)
    lay[0, nt[:, 0], nt[:, 1]] = 1
    return lay


# program -> (nb, bs, generator or None, mask predicate, ctx)
CASES = {
    "stride_fusion_test": (32, 32, ("sawtooth", dict(chunks=1)), "causal_all", 0),
    "local_fusion_test": (32, 32, ("local", dict(left=1, right=0)), "local", 32),
    "no_fusion_test": (10, 32, ("full", dict(causal=1)), "causal_diag", 0),
    "big_bird_fusion_test": (10, 32, None, None, 0),
}


@pytest.mark.parametrize("prog", sorted(CASES))
def test_lut_and_mask_match_reference_uploads(oracle, prog):
    g = np.load(os.path.join(GOLD, "ref_uploads.npz"))
    nb, bs, gen, pred, ctx = CASES[prog]
    nt_ref = g[prog + "/nt_lut"].reshape(-1, 2)
    lay = _layout_from_nt(nt_ref, nb)
    if gen is not None:
        assert np.array_equal(oracle.layout(gen[0], 1, nb, **gen[1]), lay)
    luts = oracle.lut_build(lay)
    assert np.array_equal(luts["nt"][0], nt_ref)
    assert np.array_equal(luts["nn"][0], g[prog + "/nn_lut"].reshape(-1, 2))
    if prog + "/rblk_lut" in g:
        assert np.array_equal(luts["rblk"][0], g[prog + "/rblk_lut"].reshape(-1, 2))
    if pred is not None:
        code = dict(causal_all=oracle.MASK_CAUSAL_ALL, causal_diag=oracle.MASK_CAUSAL_DIAG,
                    local=oracle.MASK_LOCAL)[pred]
        m_np, m_t = oracle.mask_pack(luts["nt"], bs, code, ctx)
        assert np.array_equal(m_np.ravel(), g[prog + "/mask_np"])
        assert np.array_equal(m_t.ravel(), g[prog + "/mask_t"])


@pytest.mark.parametrize("prog", sorted(CASES))
def test_nn_max_matches_reference_softmax_launch(oracle, prog):
    """The reference sizes the softmax CTA from nn_max (blocksparse.h:665-680): threads =
    ceil(nn_max*bs/256)*32, shared = threads*4/16*8 bytes; grid = (L, B, H)."""
    g = np.load(os.path.join(GOLD, "ref_uploads.npz"))
    nb, bs, _, _, _ = CASES[prog]
    luts = oracle.lut_build(_layout_from_nt(g[prog + "/nt_lut"].reshape(-1, 2), nb))
    line = [l for l in g[prog + "/launches"] if "bst_masked_softmax" in l][0].split()
    grid_x, threads, smem = int(line[1]), int(line[4]), int(line[7])
    want_threads = -(-luts["nn_max"] * bs // 256) * 32
    assert grid_x == nb * bs
    assert threads == want_threads
    assert smem == (want_threads * 4 >> 4) * 8
    sddmm = [l for l in g[prog + "/launches"] if "bst_sgemm_32x32x64_nt" in l][0].split()
    assert int(sddmm[1]) == luts["blocks"]


def test_attention_matches_reference_cpu_operators(oracle):
    g = np.load(os.path.join(GOLD, "ref_cpu_attention.npz"))
    B, L, H, d = (int(x) for x in g["attn/shape"])
    sq, sk, sv = (int(x) for x in g["attn/seeds"])
    bs = 32
    nb = L // bs
    q, k, v = (oracle.fill_normal((B, L, H, d), s) for s in (sq, sk, sv))
    luts = oracle.lut_build(oracle.layout("full", 1, nb, causal=1))
    m_np, _ = oracle.mask_pack(luts["nt"], bs, oracle.MASK_CAUSAL_DIAG)
    r = oracle.attention(q, k, v, luts, bs, np.float32(1.0 / np.sqrt(d)), mask_np=m_np)
    tri = np.tril(np.ones((L, L), bool))
    s = oracle.blocks_to_dense(r["s"], luts["nt"], nb, bs)
    p = oracle.blocks_to_dense(r["p"], luts["nt"], nb, bs)
    # bit-exact: same operation order as matmul.h / ewops.h
    assert np.array_equal(np.where(tri, s, 0), g["attn/s"])
    assert np.array_equal(p, g["attn/p"])
    assert np.array_equal(r["o"], g["attn/o"])


def test_attention_matches_live_reference_when_built(oracle):
    if oracle.ref() is None:
        pytest.skip("oracle/_ref not built on this machine")
    B, L, H, d, bs = 1, 128, 2, 32, 64
    q, k, v = (oracle.fill_normal((B, L, H, d), s) for s in (5, 6, 7))
    luts = oracle.lut_build(oracle.layout("full", 1, L // bs, causal=1))
    m_np, _ = oracle.mask_pack(luts["nt"], bs, oracle.MASK_CAUSAL_DIAG)
    r = oracle.attention(q, k, v, luts, bs, 0.25, mask_np=m_np)
    s, p, o = oracle.ref_dense_causal_attention(q, k, v, 0.25)
    assert np.array_equal(oracle.blocks_to_dense(r["p"], luts["nt"], L // bs, bs), p)
    assert np.array_equal(r["o"], o)


def test_layernorm_matches_reference_cpu_operators(oracle):
    g = np.load(os.path.join(GOLD, "ref_cpu_attention.npz"))
    m, hidden = (int(x) for x in g["ln/shape"])
    sx, sr, sb, sg, sbe = (int(x) for x in g["ln/seeds"])
    x = oracle.fill_normal((m, hidden), sx)
    r = oracle.fill_normal((m, hidden), sr)
    b = oracle.fill_normal((hidden,), sb, 0.02)
    gain = 1.0 + oracle.fill_normal((hidden,), sg, 0.1)
    beta = oracle.fill_normal((hidden,), sbe, 0.1)
    y, summed, mean, rstd = oracle.bias_residual_layernorm(x, b, r, gain, beta)
    assert np.array_equal(summed, g["ln/sum"])
    assert np.array_equal(mean, g["ln/mean"])
    assert np.array_equal(rstd, g["ln/rstd"])
    assert np.array_equal(y, g["ln/y"])


@pytest.mark.parametrize("kind,kw,H", [("fixed", dict(stride=4), 4), ("local", dict(left=1, right=0), 1),
                                         ("bigbird", dict(nrand=3), 1)])
def test_all_ones_known_answer(oracle, kind, kw, H):
    B, L, d, bs = 1, 256, 128, 32
    nb = L // bs
    luts = oracle.lut_build(oracle.layout(kind, H, nb, **kw))
    ones = np.ones((B, L, H, d), np.float32)
    r = oracle.attention(ones, ones, ones, luts, bs, np.float32(1 / np.sqrt(d)), eps=0.0)
    assert np.all(r["s"] == d)
    for h in range(H):
        nn = luts["nn"][h]
        for i in range(nb):
            cnt = int(nn[i, 1])
            for e in range(cnt):
                blk = int(nn[int(nn[i, 0]) + e, 0])
                np.testing.assert_allclose(r["p"][0, h, blk], 1.0 / (cnt * bs), rtol=1e-6)
    np.testing.assert_allclose(r["o"], 1.0, rtol=1e-5)


def test_layout_block_counts():
    """Block counts of the five benchmark configurations."""
    import oracle_lib as O
    assert O.lut_build(O.layout("fixed", 4, 16, stride=4))["blocks"] == 112
    st = O.lut_build(O.layout("stride", 1, 64, band=4, every=8))
    assert (st["blocks"], st["nn_max"]) == (730, 12)
    lo = O.lut_build(O.layout("local", 1, 256, left=8, right=8))
    assert (lo["blocks"], lo["nn_max"]) == (4280, 17)
    fu = O.lut_build(O.layout("full", 1, 16))
    assert (fu["blocks"], fu["nn_max"]) == (256, 16)
    bb = O.lut_build(O.layout("bigbird", 1, 64, window=1, g_first=1, g_last=1, nrand=3, seed=1236))
    assert bb["nn_max"] == 64 and 560 <= bb["blocks"] <= 620


def test_magicu64_divides(oracle):
    for d in (1, 2, 3, 4, 5, 7, 8, 12):
        magic, shift = oracle.magicu64(d)
        for n in (0, 1, d - 1, d, 5 * d + 3, 1000, 65535):
            got = n >> shift if magic == 1 else ((n * magic) >> 32) >> shift
            assert got == n // d


def test_to_bhalf_rounds_half_away(oracle):
    below = np.nextafter(np.float32(1.00390625), np.float32(0))
    v = np.array([1.0, 1.00390625, below, 1.0117188, -1.00390625, 0.0, 3.0e38], np.float32)
    bits = oracle.to_bhalf(v)
    assert list(bits[:5]) == [0x3F80, 0x3F81, 0x3F80, 0x3F82, 0xBF81]


def test_gelu_matches_live_reference_when_built(oracle):
    if oracle.ref() is None:
        pytest.skip("oracle/_ref not built on this machine")
    x = oracle.fill_normal((7, 96), 41, 2.0)
    b = oracle.fill_normal((96,), 42, 0.5)
    assert np.array_equal(oracle.bias_gelu(x, b), oracle.ref_bias_gelu(x, b))


def test_tn_lut_matches_reference_generator():
    """generate_tn_lut (ewops.h:675-701; inlined in test.cu:139-170) writes, for the dense causal
    layout, header[c] = (running offset starting at nb, nb - c) and entries (row*(row+1)/2 + col, row)
    column by column.  The layout-driven builder must reproduce exactly that."""
    import oracle_lib as O
    nb = 10
    got = O.lut_build_tn(O.layout("full", 1, nb, causal=1))
    blocks = nb * (nb + 1) // 2
    want = np.zeros((nb + blocks, 2), np.uint32)
    total, cnt = nb, nb
    for c in range(nb):
        want[c] = (total, cnt)
        total += cnt
        cnt -= 1
    at = nb
    for col in range(nb):
        for row in range(col, nb):
            want[at] = (row * (row + 1) // 2 + col, row)
            at += 1
    assert got["blocks"] == blocks and got["tn_max"] == nb
    assert np.array_equal(got["tn"][0], want)


@pytest.mark.parametrize("kind,kw", [("stride", dict(band=4, every=8)), ("bigbird", dict(window=1, g_first=1, g_last=1, nrand=3, seed=7)),
                                     ("fixed", dict(stride=4))])
def test_tn_lut_is_the_transpose_of_nn_lut(kind, kw):
    """Every block appears once in each LUT with the same id; tn walks columns, nn walks rows."""
    import oracle_lib as O
    heads, nb = (4, 16) if kind == "fixed" else (1, 16)
    lay = O.layout(kind, heads, nb, **kw)
    nn, tn = O.lut_build(lay), O.lut_build_tn(lay)
    for h in range(heads):
        seen = {}
        for i in range(nb):
            off, cnt = nn["nn"][h, i]
            for e in range(cnt):
                blk, col = nn["nn"][h, off + e]
                seen[int(blk)] = (i, int(col))
        back = {}
        for j in range(nb):
            off, cnt = tn["tn"][h, j]
            rows = [int(tn["tn"][h, off + e, 1]) for e in range(cnt)]
            assert rows == sorted(rows)
            for e in range(cnt):
                blk, row = tn["tn"][h, off + e]
                back[int(blk)] = (int(row), j)
        assert seen == back and len(seen) == nn["blocks"]
        assert tn["tn_max"] == int(lay.sum(axis=1).max())


def test_backward_matches_reference_cpu_operators(oracle):
    """softmax grad, TN and NN products of the oracle against the reference's own CPU operators on the
    dense causal layout (fixture made by tests/golden/make_golden.py): bit-exact, same operation order."""
    g = np.load(os.path.join(GOLD, "ref_cpu_backward.npz"))
    B, L, H, d = (int(x) for x in g["bwd/shape"])
    q, k, v, do = (oracle.fill_normal((B, L, H, d), int(s)) for s in g["bwd/seeds"])
    bs, nb = 32, L // 32
    lay = oracle.layout("full", 1, nb, causal=1)
    luts, tn = oracle.lut_build(lay), oracle.lut_build_tn(lay)["tn"]
    scale = np.float32(1.0 / np.sqrt(d))

    def to_blocks(dense):          # [B,H,L,L] -> [B,H,blocks,bs,bs]
        out = np.zeros((B, H, luts["blocks"], bs, bs), np.float32)
        for kk, (i, j) in enumerate(luts["nt"][0]):
            out[:, :, kk] = dense[:, :, i * bs:(i + 1) * bs, j * bs:(j + 1) * bs]
        return out

    bhld = lambda a: a.transpose(0, 2, 1, 3)    # [B,H,L,d] <-> [B,L,H,d]
    p_blk = to_blocks(g["bwd/p"])
    # dP = dO V^T on the kept blocks: the scores of the forward oracle with (q, k) := (dO, V)
    dp = oracle.attention(do, v, v, luts, bs, scale, want=("s",))["s"]
    tri = np.tril(np.ones((L, L), bool))
    assert np.array_equal(np.where(tri, oracle.blocks_to_dense(dp, luts["nt"], nb, bs), 0), np.where(tri, g["bwd/dp"], 0))
    # dV = P^T dO
    assert np.array_equal(bhld(oracle.spmm_tn(p_blk, do, tn, bs)), g["bwd/dv"])
    # dS: the reference sums dy*y over the whole dense row; the products outside the triangle are exact zeros
    ds = oracle.softmax_grad(to_blocks(g["bwd/dp"]), p_blk, luts, bs, scale)
    assert np.array_equal(oracle.blocks_to_dense(ds, luts["nt"], nb, bs), g["bwd/ds"])
    # dQ = dS K, dK = dS^T Q
    assert np.array_equal(bhld(oracle.spmm_nn(ds, k, luts["nn"], bs)), g["bwd/dq"])
    assert np.array_equal(bhld(oracle.spmm_tn(ds, q, tn, bs)), g["bwd/dk"])


def test_linear_matches_live_reference_when_built(oracle):
    """orc_linear against the reference's matrixMulNNCPU (+ its bias and gelu, pinned above) -- bit-exact."""
    if oracle.ref() is None:
        pytest.skip("oracle/_ref not built on this machine")
    x = oracle.fill_normal((37, 72), 51)
    w = oracle.fill_normal((72, 48), 52, 0.02)
    b = oracle.fill_normal((48,), 53, 0.1)
    plain = oracle.ref_matmul_nn(x, w)
    assert np.array_equal(oracle.linear(x, w), plain)
    assert np.array_equal(oracle.linear(x, w, b, act=1), oracle.ref_bias_gelu(plain, b))


def test_embedding_and_logits_match_live_reference_when_built(oracle):
    """orc_embedding against embedding_lookup + tensor_add_matrix, orc_linear_nt against matrixMulNTCPU -- bit-exact."""
    if oracle.ref() is None:
        pytest.skip("oracle/_ref not built on this machine")
    vocab, hidden, B, L = 97, 40, 3, 17
    table = oracle.fill_normal((vocab, hidden), 61, 0.02)
    pos = oracle.fill_normal((L, hidden), 62, 0.02)
    ids = (np.arange(B * L, dtype=np.int64) * 37 % vocab).astype(np.int32).reshape(B, L)
    assert np.array_equal(oracle.embedding(table, ids, pos), oracle.ref_embedding(table, ids, pos))
    x = oracle.fill_normal((B * L, hidden), 63)
    assert np.array_equal(oracle.linear_nt(x, table), oracle.ref_matmul_nt(x, table))
    bad = ids.copy()
    bad[0, 0], bad[1, 2] = -1, vocab
    out = oracle.embedding(table, bad, None)
    assert float(np.abs(out[0, 0]).max()) == 0.0 and float(np.abs(out[1, 2]).max()) == 0.0


def test_csr_path_matches_live_reference_when_built(oracle):
    """The CSR causal pattern against generate_csr_full_mask, and CSR attention on it against the reference's dense
    causal CPU attention (the one pattern both can express) -- bit-exact."""
    if oracle.ref() is None:
        pytest.skip("oracle/_ref not built on this machine")
    L = 48
    rowptr, colidx = oracle.csr_full_mask(L)
    rr, rc = oracle.ref_csr_full_mask(2, 3, L)
    nnz = L * (L + 1) // 2
    for g in range(6):      # the reference stacks one copy per (batch, head), row pointers running on
        assert np.array_equal(rr[g * L:(g + 1) * L + 1] - g * nnz, rowptr)
        assert np.array_equal(rc[g * nnz:(g + 1) * nnz], colidx)
    q, k, v = (oracle.fill_normal((2, L, 3, 16), s) for s in (71, 72, 73))
    o = oracle.csr_attention(q, k, v, rowptr, colidx, 0.25)
    _, _, want = oracle.ref_dense_causal_attention(q, k, v, 0.25)
    assert np.array_equal(o, want)


def test_csr_attention_equals_block_attention_on_a_block_pattern(oracle):
    bs, nb = 32, 6
    lay = oracle.layout("stride", 1, nb, band=2, every=3)
    luts = oracle.lut_build(lay)
    rowptr, colidx = oracle.csr_from_layout(lay[0], bs)
    q, k, v = (oracle.fill_normal((1, nb * bs, 2, 32), s) for s in (81, 82, 83))
    a = oracle.attention(q, k, v, luts, bs, 0.2, want=("o",))["o"]
    b = oracle.csr_attention(q, k, v, rowptr, colidx, 0.2)
    assert np.array_equal(a, b)

