"""The `rptc` / `rptc_lite` modules (reference function names) against the golden vectors produced by
the reference's own code: the encoder on CPU, the decoder (CUDA kernels) in the GPU-marked tests."""
import numpy as np
import pytest
import torch


def test_rptc_quantize_matches_reference_encoder(golden):
    import rptc
    alphabet = torch.from_numpy(golden["enc8_alphabet"])
    for s, want_q, want_loss in zip(golden["enc8_samples"], golden["enc8_symbols"], golden["enc8_loss"]):
        q, loss = rptc.quantize(alphabet, torch.eye(len(s)), torch.from_numpy(s))
        assert np.array_equal(q.numpy(), want_q)
        assert abs(float(loss) - want_loss) <= 1e-5 * max(1.0, abs(want_loss))


def test_rptc_lite_quantize_and_index_match_reference(golden):
    import rptc_lite
    assert np.array_equal(rptc_lite.index_fn(torch.from_numpy(golden["c_index_states"]), 16, 9).numpy(), golden["c_index"])
    alphabet = torch.from_numpy(golden["encc_alphabet"])
    for s, want_q, want_loss in zip(golden["encc_samples"], golden["encc_symbols"], golden["encc_loss"]):
        q, loss = rptc_lite.quantize(alphabet, 8, 5, 4, torch.ones(s.shape), torch.from_numpy(s))
        assert np.array_equal(q.numpy(), want_q)
        assert abs(float(loss) - want_loss) <= 1e-5 * max(1.0, abs(want_loss))


def test_pack_symbols_matches_oracle():
    import rptc
    import rptc_oracle as o
    rng = np.random.default_rng(0)
    for bits, T in ((2, 100), (4, 37), (8, 16)):
        sym = rng.integers(0, 1 << bits, (3, T))
        got = rptc.pack_symbols(torch.from_numpy(sym), bits).numpy().view(np.uint32)
        assert np.array_equal(got, o.pack_symbols(sym, bits))


def test_dequantize_refuses_cpu_tensors():
    import rptc
    with pytest.raises(RuntimeError):
        rptc.dequantize(torch.zeros(65536), torch.zeros(16, dtype=torch.int32))


@pytest.mark.gpu
def test_rptc_dequantize_on_gpu_matches_reference(golden):
    import rptc
    for L in (16, 14):
        alphabet = torch.from_numpy(golden[f"a{L}_alphabet"]).cuda()
        sym = torch.from_numpy(golden[f"a{L}_symbols"]).cuda()
        got = rptc.dequantize(alphabet, sym)
        want = golden[f"a{L}_decoded"].astype(np.float16).astype(np.float32)       # fp16 codebook on the device
        assert np.array_equal(got.cpu().numpy(), want)
        assert np.array_equal(rptc.dequantize(alphabet, sym[0]).cpu().numpy(), want[0])


@pytest.mark.gpu
def test_rptc_lite_dequantize_on_gpu_matches_reference(golden):
    import rptc_lite
    alphabet = torch.from_numpy(golden["c_alphabet"]).cuda()
    sym = torch.from_numpy(golden["c_symbols"]).cuda()
    got = rptc_lite.dequantize(alphabet, 16, 9, 4, sym)
    want = golden["c_decoded"].astype(np.float16).astype(np.float32)
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.gpu
def test_config0_quantize_pack_decompress_matvec():
    """BASELINE config 0 in small: rows of iid N(0,1) weights, quantised with the reference's trellis
    (L = 16 state bits, K = 2), then decompress + matvec on the GPU."""
    import rptc
    from rptc_b200 import CODE_LUT, LAYOUT_ROWMAJOR, LAYOUT_TILED, Format, ops
    from rptc_b200.linear import gaussian_codebook
    g = torch.Generator(device="cuda").manual_seed(42)
    m, n = 32, 1024
    W = torch.randn((m, n), device="cuda", generator=g)
    fmt = Format(CODE_LUT, 2, 16, 0, LAYOUT_TILED)
    alphabet = gaussian_codebook(fmt, g, "cuda").float()
    q, loss = rptc.quantize_rows(alphabet, torch.ones(n, device="cuda"), W)
    recon = rptc.dequantize(alphabet, q)
    mse = ((recon - W) ** 2).mean().item()
    assert abs(loss.sum().item() / (m * n) - mse) < 5e-3           # the encoder's own loss is the decode error
    assert mse < 0.12                                              # 2-bit TCQ of a unit Gaussian (scalar Lloyd-Max is 0.1175)
    words = rptc.pack_symbols(q, 2)
    codes = ops.repack(words.contiguous(), LAYOUT_ROWMAJOR, LAYOUT_TILED, m, n // 64)
    x = torch.randn((1, n), dtype=torch.float16, device="cuda", generator=g)
    y = ops.gemv(codes, alphabet.half(), x, m, n, fmt).float()
    ref = x.float() @ recon.t()
    assert (y - ref).abs().max() <= 2e-3 * recon.norm(dim=1).max() * x.float().norm() + 1e-2
