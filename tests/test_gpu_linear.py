"""GPU parity of the tcgen05 dense projection (sfb_linear, sfb_linear_nt) and of the embedding front end against the CPU oracle.  Tolerance: 16-bit operands with
fp32 accumulation, 2e-2 relative to the largest reference value (the output itself is rounded to 16 bits)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TD = {"bf16": torch.bfloat16, "f16": torch.float16}


def _mk(oracle, shape, seed, dtype, std=1.0):
    t = torch.from_numpy(oracle.fill_normal(shape, seed, std)).cuda().to(TD[dtype])
    return t, t.float().cpu().numpy()


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("m,n,k,act,with_bias", [
    (128, 256, 64, 0, False),        # one tile, one k-block
    (128, 256, 768, 0, True),
    (300, 768, 768, 0, True),        # ragged rows, three column tiles
    (257, 3072, 768, 1, True),       # FFN up-projection with GELU
    (130, 768, 3072, 0, True),       # FFN down-projection: 48 k-blocks
    (64, 48, 40, 1, True),           # smaller than a tile in every direction; k not a multiple of 64
    (1000, 1024, 1024, 0, False),
])
def test_linear_against_oracle(sfb, oracle, dtype, m, n, k, act, with_bias):
    x, xn = _mk(oracle, (m, k), 400, dtype)
    w, wn = _mk(oracle, (k, n), 401, dtype, 0.05)
    b = torch.from_numpy(oracle.fill_normal((n,), 402, 0.5)).cuda() if with_bias else None
    got = sfb.linear(x, w, b, act)
    assert sfb.device_status() == 0
    want = oracle.linear(xn, wn, None if b is None else b.cpu().numpy(), act)
    assert got.shape == (m, n) and got.dtype == TD[dtype]
    assert np.abs(got.float().cpu().numpy() - want).max() <= 2e-2 * np.abs(want).max()


def test_linear_more_tiles_than_sms_and_batched_input(sfb, oracle):
    """A [B, L, hidden] activation (leading dimensions flattened) with enough tiles that every CTA loops."""
    B, L, hidden, n = 2, 4096, 768, 2304
    x = torch.randn(B, L, hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)).to(torch.bfloat16)
    w = (0.05 * torch.randn(hidden, n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(10))).to(torch.bfloat16)
    b = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(11))
    got = sfb.linear(x, w, b)
    assert sfb.device_status() == 0 and got.shape == (B, L, n)
    # rows sampled across all tiles against the oracle; everything against a float32 matmul on the device
    rows = np.arange(0, B * L, 97)
    want = oracle.linear(x.view(-1, hidden)[rows].float().cpu().numpy(), w.float().cpu().numpy(), b.cpu().numpy())
    assert np.abs(got.view(-1, n)[rows].float().cpu().numpy() - want).max() <= 2e-2 * np.abs(want).max()
    full = x.view(-1, hidden).float() @ w.float() + b
    assert float((got.view(-1, n).float() - full).abs().max()) <= 2e-2 * float(full.abs().max())


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("m,n,k,act,transposed", [
    (19000, 256, 64, 0, False),      # one k-block, one column tile, every pair of CTAs busy
    (2500, 2320, 200, 1, False),     # ragged in m (last 256-row tile: 196 rows), n (16 columns into the last tile) and k
    (4096, 768, 3072, 0, False),     # 48 k-blocks: the stage ring wraps eight times per tile
    (2304, 4000, 512, 1, True),      # w as [n, k]; the odd CTA's half of the last column tile lies beyond n
    (129, 19200, 128, 0, True),      # a single row into the second CTA's half
    (8192, 768, 256, 0, True),
    (8192, 752, 200, 1, True),       # ragged n (the last tile's second half has 112 of its 128 columns) and k
])
def test_linear_on_cta_pairs(sfb, dtype, m, n, k, act, transposed):
    """Shapes with at least one 256 x 256 tile per pair of SMs take the two-CTA kernel: against a float32 product on
    the device (the oracle checks the same entry point on small shapes above)."""
    gen = torch.Generator(device="cuda").manual_seed(77)
    x = torch.randn(m, k, device="cuda", generator=gen).to(TD[dtype])
    w = (0.05 * torch.randn(k, n, device="cuda", generator=gen)).to(TD[dtype])
    b = torch.randn(n, device="cuda", generator=gen)
    got = sfb.linear_nt(x, w.t().contiguous(), b, act) if transposed else sfb.linear(x, w, b, act)
    assert sfb.device_status() == 0
    t = x.float() @ w.float() + b
    want = t * torch.sigmoid(1.702 * t) if act else t
    assert got.shape == (m, n)
    assert float((got.float() - want).abs().max()) <= 2e-2 * float(want.abs().max())


def test_linear_rejects_what_it_cannot_do(sfb):
    x = torch.zeros(16, 64, device="cuda")
    w = torch.zeros(64, 64, device="cuda")
    with pytest.raises(sfb.SfbError):
        sfb.linear(x, w)                                   # fp32
    xb, wb = x.to(torch.bfloat16), torch.zeros(64, 24, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(sfb.SfbError):
        sfb.linear(xb, wb)                                 # n not a multiple of 16


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("m,n,k,act", [(128, 256, 64, 0), (300, 1008, 768, 0), (257, 30528, 1024, 0), (64, 48, 40, 1)])
def test_linear_nt_against_oracle(sfb, oracle, dtype, m, n, k, act):
    """out = x . wt^T with wt [n, k] -- the logits over a (padded) tied embedding table."""
    x, xn = _mk(oracle, (m, k), 410, dtype)
    wt, wn = _mk(oracle, (n, k), 411, dtype, 0.05)
    b = torch.from_numpy(oracle.fill_normal((n,), 412, 0.5)).cuda()
    got = sfb.linear_nt(x, wt, b, act)
    assert sfb.device_status() == 0
    rows = np.arange(0, m, max(1, m // 40))
    want = oracle.linear_nt(xn[rows], wn, b.cpu().numpy(), act)
    assert got.shape == (m, n) and got.dtype == TD[dtype]
    assert np.abs(got[rows].float().cpu().numpy() - want).max() <= 2e-2 * np.abs(want).max()
    # the transposed-weight path and the plain one are the same product
    same = sfb.linear(x, wt.t().contiguous(), b, act)
    assert float((got.float() - same.float()).abs().max()) <= 2e-2 * float(same.float().abs().max())


@pytest.mark.parametrize("dtype,hidden", [("f32", 768), ("bf16", 1024), ("f16", 40)])
def test_embedding_bit_exact(sfb, oracle, dtype, hidden):
    td = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    vocab, B, L = 3000, 3, 257
    table = torch.from_numpy(oracle.fill_normal((vocab, hidden), 420, 0.02)).cuda().to(td)
    pos = torch.from_numpy(oracle.fill_normal((L, hidden), 421, 0.02)).cuda().to(td)
    ids = torch.from_numpy((np.arange(B * L, dtype=np.int64) * 7919 % vocab).astype(np.int32).reshape(B, L)).cuda()
    out, bad = sfb.embedding(table, ids, pos)
    assert int(bad.item()) == 0
    want = oracle.embedding(table.float().cpu().numpy(), ids.cpu().numpy(), pos.float().cpu().numpy())
    if dtype == "f32":
        assert np.array_equal(out.cpu().numpy(), want)
    else:   # one rounding of the sum to 16 bits
        assert np.array_equal(out.float().cpu().numpy(), torch.from_numpy(want).to(td).float().numpy())
    plain, _ = sfb.embedding(table, ids)
    assert torch.equal(plain, table[ids.long()])


@pytest.mark.parametrize("B,L,hidden", [(37, 8, 64), (5, 2, 1024), (130, 33, 128), (1, 4096, 768)])
def test_embedding_batch_runs(sfb, B, L, hidden):
    """A thread keeps one piece of a position row for a run of batch elements; short sequences split the batch over
    the grid.  Batches that are no multiple of the run length or of the steps inside it, and a batch of one."""
    gen = torch.Generator(device="cuda").manual_seed(31)
    vocab = 1000
    table = torch.randn(vocab, hidden, device="cuda", generator=gen).to(torch.bfloat16)
    pos = torch.randn(L, hidden, device="cuda", generator=gen).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (B, L), device="cuda", generator=gen, dtype=torch.int32)
    ids[B // 2, L // 2] = vocab + 3          # one id outside the table: zeros + position, counted once
    out, bad = sfb.embedding(table, ids, pos)
    assert int(bad.item()) == 1
    rows = table[ids.clamp(0, vocab - 1).long()].float()
    rows[B // 2, L // 2] = 0.0
    want = (rows + pos.float().unsqueeze(0)).to(torch.bfloat16)
    assert torch.equal(out, want)


def test_embedding_ids_outside_the_table_are_counted_not_read(sfb):
    table = torch.ones(10, 16, device="cuda", dtype=torch.bfloat16)
    ids = torch.tensor([[0, 9, 10, -1, 5]], dtype=torch.int32, device="cuda")
    out, bad = sfb.embedding(table, ids)
    assert int(bad.item()) == 2
    assert out[0, :, 0].float().cpu().tolist() == [1.0, 1.0, 0.0, 0.0, 1.0]

