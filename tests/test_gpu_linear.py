"""GPU parity of the tcgen05 dense projection (sfb_linear) against the CPU oracle.  Tolerance: 16-bit operands with
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


def test_linear_rejects_what_it_cannot_do(sfb):
    x = torch.zeros(16, 64, device="cuda")
    w = torch.zeros(64, 64, device="cuda")
    with pytest.raises(sfb.SfbError):
        sfb.linear(x, w)                                   # fp32
    xb, wb = x.to(torch.bfloat16), torch.zeros(64, 24, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(sfb.SfbError):
        sfb.linear(xb, wb)                                 # n not a multiple of 16
