"""The CUDA trellis encoder (csrc/viterbi.cu) against the reference's own encoder output (golden vectors), against
the torch restatement on the CPU, and on BASELINE's single-linear case: Gaussian weights encoded at L = 16, packed,
decoded and multiplied on the GPU."""
import numpy as np
import pytest
import torch

import rptc_oracle as o

pytestmark = pytest.mark.gpu


def test_cuda_encoder_reproduces_the_reference_encoder(golden):
    import rptc
    alphabet = torch.from_numpy(golden["enc8_alphabet"]).cuda()
    samples = torch.from_numpy(golden["enc8_samples"]).cuda()
    weights = torch.ones(samples.shape[1], device="cuda")
    sym, loss = rptc.quantize_rows(alphabet, weights, samples)
    assert sym.dtype == torch.int32
    assert np.array_equal(sym.cpu().numpy(), golden["enc8_symbols"])
    np.testing.assert_allclose(loss.cpu().numpy(), golden["enc8_loss"], rtol=1e-5)


@pytest.mark.parametrize("L,n,rows,ties", [(4, 9, 3, False), (6, 40, 5, False), (10, 130, 9, False), (8, 64, 6, True), (12, 50, 130, False)])
def test_cuda_encoder_matches_the_cpu_recurrence(L, n, rows, ties):
    import rptc
    g = torch.Generator().manual_seed(L * 100 + n)
    alphabet = torch.randn(1 << L, generator=g)
    if ties:
        alphabet = (alphabet * 2).round() / 2             # few distinct values: equal costs everywhere, first minimum wins
    samples = torch.randn(rows, n, generator=g)
    if ties:
        samples = (samples * 2).round() / 2
    weights = 0.5 + torch.rand(n, generator=g)
    want_sym, want_loss = rptc.quantize_rows(alphabet, weights, samples)               # torch, on the CPU
    got_sym, got_loss = rptc.quantize_rows(alphabet.cuda(), weights.cuda(), samples.cuda())
    assert torch.equal(got_sym.cpu(), want_sym)
    torch.testing.assert_close(got_loss.cpu(), want_loss, rtol=1e-5, atol=1e-6)
    # the symbols walk the trellis to the cost the encoder reports
    for r in range(min(rows, 3)):
        dec = o.dequantize_symbols(alphabet.numpy(), want_sym[r].numpy())
        cost = float((weights.numpy().astype(np.float64) * (samples[r].numpy().astype(np.float64) - dec) ** 2).sum())
        assert abs(cost - float(got_loss[r])) <= 1e-4 * max(1.0, cost)


def test_single_linear_gaussian_weights_at_L16():
    """BASELINE's single-linear case at 256 x 4096: N(0,1) weights, Gaussian-quantile alphabet in a seeded random order,
    encoded at L = 16 / 2 bits per weight, packed, decoded bit-exactly and multiplied by one fp16 vector."""
    import rptc
    from rptc_b200 import CODE_LUT, LAYOUT_ROWMAJOR, LAYOUT_TILED, Format, ops
    m, n, L = 256, 4096, 16
    g = torch.Generator(device="cuda").manual_seed(42)
    W = torch.randn(m, n, generator=g, device="cuda")
    M = 1 << L
    q = (2 * torch.arange(M, dtype=torch.float64, device="cuda") + 1) / (2 * M)
    alphabet = (2.0 ** 0.5 * torch.erfinv(2 * q - 1)).float()[torch.randperm(M, generator=g, device="cuda")]      # rptc.py:143-146
    sym, loss = rptc.quantize_rows(alphabet, torch.ones(n, device="cuda"), W)
    assert int(sym.min()) >= 0 and int(sym.max()) <= 3
    W_hat = rptc.dequantize(alphabet, sym)                                            # CUDA decompress of the packed symbols
    mse = float(((W - W_hat.float()) ** 2).mean())
    assert 0.06 < mse < 0.09, mse                      # 2 bits per weight: the distortion-rate bound is 0.0625
    torch.testing.assert_close(loss / n, ((W - alphabet[_states(sym, L)]) ** 2).mean(dim=1), rtol=1e-4, atol=1e-5)
    lut16 = alphabet.half()
    for r in (0, 17, m - 1):                           # bit-exact against the oracle's sequential decode
        want = o.dequantize_symbols(lut16.cpu().numpy(), sym[r].cpu().numpy())
        assert np.array_equal(W_hat[r].half().cpu().numpy().view(np.uint16), want.view(np.uint16))
    words = rptc.pack_symbols(sym)
    fmt = Format(CODE_LUT, 2, L, 0, LAYOUT_TILED)
    codes = ops.repack(words.contiguous(), LAYOUT_ROWMAJOR, LAYOUT_TILED, m, n // 64)
    x = torch.randn(n, generator=g, device="cuda").half()
    y = ops.gemv(codes, lut16, x, m, n, fmt).float()
    want = W_hat.half().float() @ x.float()
    assert (y - want).abs().max().item() <= 2e-3 * float(W_hat.float().norm(dim=1).max() * x.float().norm())


def _states(sym: torch.Tensor, L: int) -> torch.Tensor:
    """The state visited at every position of every row (the last L bits of the symbol stream)."""
    state = torch.zeros(sym.shape[0], dtype=torch.int64, device=sym.device)
    out = torch.empty(sym.shape, dtype=torch.int64, device=sym.device)
    for i in range(sym.shape[1]):
        state = ((state << 2) | sym[:, i].long()) & ((1 << L) - 1)
        out[:, i] = state
    return out
