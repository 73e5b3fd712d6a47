"""The HF driver's layer functions against vectors produced by the reference's own quantize_hf.py
(tests/golden/make_golden.py), and the packed layer / model swap on the GPU."""
import numpy as np
import pytest
import torch

import rptc_oracle as o


def _np_permute(key):
    def permute(alphabet):
        return alphabet[torch.from_numpy(np.random.default_rng(key).permutation(alphabet.numel())).to(alphabet.device)]
    return permute


def test_factorize_matches_reference(golden):
    import quantize_hf as q
    parts = q.factorize(torch.from_numpy(golden["fact_W"]))
    for name, got in zip(("biases_out", "biases_in", "scales_out", "scales_in", "normalized"), parts):
        np.testing.assert_allclose(got.numpy(), golden[f"fact_{name}"], rtol=2e-4, atol=2e-5, err_msg=name)
    bo, bi, so, si, nz = parts
    np.testing.assert_allclose((bo + bi + so * si * nz).numpy(), golden["fact_W"], rtol=1e-5, atol=1e-5)


def test_evaluate_layer_matches_reference(golden):
    import quantize_hf as q
    got = q.evaluate_layer(*(torch.from_numpy(golden[k]) for k in ("eval_H", "fact_W", "eval_recon")))
    np.testing.assert_allclose([float(v) for v in got], golden["eval_metrics"], rtol=1e-4)


def test_quantize_layer_reconstruction_matches_reference(golden):
    """factorize + per-bank quantile alphabets + Viterbi rounding give the reference's reconstruction when handed
    the same alphabet permutation (L = 8, 32 banks of 8 rows)."""
    import quantize_hf as q
    W, H, key = torch.from_numpy(golden["ql_W"]), torch.from_numpy(golden["ql_H"]), int(golden["ql_key"])
    bo, bi, so, si, nz = q.factorize(W)
    symbols, alphabets = q.round_weights(_np_permute(key), nz, torch.diag(H) * si.reshape(-1), 8, num_banks=32, batch_size=8)
    per_bank = W.shape[0] // 32
    rounded = np.stack([o.dequantize_symbols(alphabets[r // per_bank].numpy(), symbols[r].numpy()) for r in range(W.shape[0])])
    recon = bo.numpy() + bi.numpy() + so.numpy() * si.numpy() * rounded
    # a row whose path differs from the reference's by a near-tie would show as an O(1) difference
    np.testing.assert_allclose(recon, golden["ql_recon"], rtol=1e-3, atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [1, 5, 40])
def test_packed_layer_forward_matches_its_reconstruction(tokens):
    import quantize_hf as q
    g = torch.Generator().manual_seed(3)
    m, n, L = 512, 256, 8
    W = (torch.randn(m, n, generator=g) * (0.5 + torch.rand(m, 1, generator=g)) + 0.1 * torch.randn(m, 1, generator=g)).cuda()
    H = torch.eye(n, device="cuda") + 0.1
    layer = q.quantize_layer(q.seeded_permute(1), H, W, L, num_banks=4, batch_size=8, bias=torch.arange(m).float() * 1e-3)
    recon = layer.reconstruct()
    frob = float(q.evaluate_layer(H, W, recon)[0])
    assert frob < 0.2 * float((W ** 2).sum() ** 0.5)            # 2 bits per weight: a small relative squared error
    x = torch.randn(tokens, n, generator=g).cuda().half()
    want = x.float() @ recon.t() + layer.bias
    got = layer(x).float()
    assert got.shape == (tokens, m)
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() <= 4e-3 * scale


@pytest.mark.gpu
def test_hf_llama_swap_and_packed_checkpoint(tmp_path):
    """A random-init Hugging Face Llama: the model with packed layers swapped in computes what the model with the
    reference's dense reconstructions computes, and survives a checkpoint round trip."""
    transformers = pytest.importorskip("transformers")
    import quantize_hf as q
    cfg = transformers.LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=4, vocab_size=128, max_position_embeddings=64)
    torch.manual_seed(0)
    dense = transformers.LlamaForCausalLM(cfg).cuda().half().eval()
    packed = transformers.LlamaForCausalLM(cfg).cuda().half().eval()
    packed.load_state_dict(dense.state_dict())
    hess = lambda layer, name: torch.eye(512 if name == "down" else 256) * (1.0 + 0.1 * layer)
    metrics = q.quantize_model(q.seeded_permute(5), packed, hess, 8, num_banks=8, batch_size=8, report=None)
    assert len(metrics) == 14 and all(0 < v[0] for v in metrics.values())
    swapped = {n: mod for n, mod in packed.named_modules() if isinstance(mod, q.FactorizedRPTCLinear)}
    assert set(swapped) == set(metrics)
    with torch.inference_mode():
        for name, mod in swapped.items():                           # what the reference's driver would have stored
            dense.get_submodule(name).weight.copy_(mod.reconstruct().half())
        ids = torch.randint(0, 128, (2, 12), device="cuda")
        want = dense(ids).logits.float()
        got = packed(ids).logits.float()
    assert (got - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    path = tmp_path / "packed.pt"
    torch.save(q.packed_checkpoint(packed), path)
    fresh = transformers.LlamaForCausalLM(cfg).cuda().half().eval()
    q.load_packed_checkpoint(fresh, torch.load(path))
    with torch.inference_mode():
        again = fresh(ids).logits.float()
    for k, v in packed.state_dict().items():
        assert torch.equal(fresh.state_dict()[k], v), k
    # same codes and tables; the matvec's partial sums meet in a different order on every launch
    assert (again - got).abs().max().item() <= 2e-3 * want.abs().max().item()


def test_packed_layer_geometry_for_llama2_7b_gate_proj_needs_no_gpu():
    """11008 rows in 32 banks is 344 rows per bank: not a multiple of 32.  The reference accepts it
    (quantize_hf.py:120-126 needs m % (num_banks * batch_size) == 0 only); the packed layer stores 11 blocks per bank."""
    import quantize_hf as q
    layer = q.FactorizedRPTCLinear(11008, 4096, 16, 32, device="cpu")
    assert layer.bank_rows == 344 and layer.bank_blocks == 11
    assert tuple(layer.codes.shape) == (32 * 11, 64, 32, 4)
    codes, lut, stored, sl = layer._bank(31)
    assert stored == 352 and codes.shape[0] == 11 and (sl.start, sl.stop) == (31 * 344, 11008)
    with pytest.raises(ValueError):
        q.FactorizedRPTCLinear(11008, 4096, 16, 33, device="cpu")


def test_packed_checkpoint_as_safetensors_needs_no_gpu(tmp_path):
    """Packed layers inside an ordinary module survive a safetensors round trip bit for bit (shapes travel as metadata)."""
    pytest.importorskip("safetensors")
    import quantize_hf as q

    def build():
        net = torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.Linear(64, 128, bias=False))
        q.swap_module(net, "0", q.FactorizedRPTCLinear(64, 64, 8, 2, True, device="cpu"))
        return net

    g = torch.Generator().manual_seed(3)
    src = build()
    for name, t in src.state_dict().items():
        if t.dtype in (torch.int32, torch.int64):
            t.copy_(torch.randint(-2**31, 2**31 - 1, t.shape, generator=g, dtype=torch.int64).to(t.dtype))
        elif t.is_floating_point():
            t.copy_(torch.randn(t.shape, generator=g).to(t.dtype))
    path = tmp_path / "packed.safetensors"
    q.save_packed_safetensors(src, path)
    dst = torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.Linear(64, 128, bias=False))       # no packed layer yet
    q.load_packed_safetensors(dst, path, device="cpu")
    assert isinstance(dst[0], q.FactorizedRPTCLinear)
    for k, v in src.state_dict().items():
        assert torch.equal(dst.state_dict()[k], v), k
    with pytest.raises(ValueError):
        from safetensors.torch import save_file
        save_file({"w": torch.zeros(2)}, str(tmp_path / "other.safetensors"))
        q.load_packed_safetensors(dst, tmp_path / "other.safetensors", device="cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [1, 12])
def test_packed_layer_with_banks_that_are_not_whole_row_blocks(tokens):
    """Llama-2-7B's gate projection height with the reference's default 32 banks, built from random symbols: the decode
    equals the oracle's row by row, and the forward pass the dense product."""
    import quantize_hf as q
    g = torch.Generator().manual_seed(9)
    m, n, L, banks = 11008, 256, 8, 32
    symbols = torch.randint(0, 4, (m, n), generator=g, dtype=torch.int32)
    alphabets = torch.randn((banks, 1 << L), generator=g)
    ones, zeros = torch.ones(m), torch.zeros(m)
    layer = q.FactorizedRPTCLinear.from_parts(symbols, alphabets, zeros, torch.zeros(n), ones, torch.ones(n))
    dec = layer.decoded().cpu().numpy()
    for r in (0, 343, 344, 5000, 11007):
        want = o.dequantize_symbols(alphabets[r // 344].numpy().astype(np.float16), symbols[r].numpy())
        assert np.array_equal(dec[r].view(np.uint16), want.view(np.uint16)), r
    x = torch.randn(tokens, n, generator=g).cuda().half()
    want = x.double() @ layer.decoded().double().t()
    got = layer(x).double()
    assert (got - want).abs().max().item() <= 2e-3 * want.abs().max().item()
