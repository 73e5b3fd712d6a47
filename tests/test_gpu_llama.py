"""GPU parity of RPTCLinear and of the Llama-shape decode engine against an fp32 torch forward of the
same network (weights decoded with the library's bit-exact decompress, transforms applied in fp32).

Tolerance (BASELINE: max-rel 1e-2 on logits): max |logit - ref| <= 1e-2 * max |ref| at every position.
"""
import numpy as np
import pytest
import torch

import rptc_oracle as o

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("code,K,S", [(o.CODE_B, 2, 8), (o.CODE_A, 2, 0), (o.CODE_C, 2, 9)])
@pytest.mark.parametrize("rows", [1, 5])
@pytest.mark.parametrize("n,m", [(4096, 1024), (11008, 512)])
def test_rptc_linear_forward_matches_effective_weight(code, K, S, rows, n, m):
    from rptc_b200 import Format
    from rptc_b200.linear import RPTCLinear
    lin = RPTCLinear.random(n, m, Format(code, K, 16, S), scale=0.02, seed=3)
    x = torch.randn((rows, n), dtype=torch.float16, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    y = lin(x).float()
    ref = x.float() @ lin.effective_weight().t()
    assert (y - ref).abs().max() <= 1e-2 * ref.abs().max()
    # the decoded matrix itself is bit-exact against the CPU oracle
    words = o.to_rowmajor(lin.codes.cpu().numpy().view(np.uint32), o.LAYOUT_TILED)
    lut = lin.lut.cpu().numpy()
    if code == o.CODE_C:
        lut = lut.reshape(-1, 2)
    ref_w = o.decode(words[:64], lut, n, code=code, K=K, L=16, S=S)
    assert np.array_equal(lin.decoded()[:64].cpu().numpy().view(np.uint16), ref_w.view(np.uint16))


def test_rptc_linear_state_dict_round_trip():
    from rptc_b200.linear import RPTCLinear
    a = RPTCLinear.random(2048, 256, seed=1)
    b = RPTCLinear.random(2048, 256, seed=2)
    b.load_state_dict(a.state_dict())
    x = torch.randn((2, 2048), dtype=torch.float16, device="cuda")
    # same codes and tables; the matvec's partial sums meet in a different order on every launch
    torch.testing.assert_close(a(x).float(), b(x).float(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("kv_heads", [2, 4])
@pytest.mark.parametrize("incoherent,hidden,ffn", [(True, 512, 1024), (False, 512, 1024), (True, 768, 1536), (True, 1024, 2816),
                                                   (True, 8192, 1024)])
def test_decode_engine_logits_match_fp32_reference(incoherent, hidden, ffn, kv_heads):
    # hidden 512 / 1024 / 8192 (two Hadamard blocks of 4096) take the fused chain, hidden 768 (not a power of two) and
    # the non-incoherent model take the unfused chain
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    # kv_heads == heads (4) takes the kernel that finishes q, k, v and attends in one launch
    cfg = LlamaConfig(hidden=hidden, layers=2, heads=4, kv_heads=kv_heads, ffn=ffn, vocab=1024, max_pos=32,
                      weight_scale=0.05 if hidden < 4096 else 0.02)
    tol = 1e-2 if hidden < 4096 else 2e-2                     # 8192-long dot products of fp16 activations
    rows, T = 2, 10
    model = RPTCLlama(cfg, rows=rows, seed=7, incoherent=incoherent)
    g = torch.Generator(device="cuda").manual_seed(11)
    tokens = torch.randint(0, cfg.vocab, (rows, T), device="cuda", generator=g)
    ref = model.reference_logits(tokens)                      # [rows, T, vocab] fp32
    for use_graph in (False, True):
        model.reset()
        if use_graph:
            model.capture(pdl=True)
        for t in range(T):
            model.ids.copy_(tokens[:, t].to(torch.int32))
            model.step()
            torch.cuda.synchronize()
            got = model.logits.float()
            err = (got - ref[:, t]).abs().max().item()
            assert err <= tol * ref[:, t].abs().max().item(), (use_graph, t, err)
        assert model.pos.tolist() == [T] * rows
    from rptc_b200 import ops
    ops.device_status()


@pytest.mark.parametrize("hidden,kv_heads", [(4096, 32), (4096, 8), (8192, 8)])
@pytest.mark.parametrize("rows", [1, 2])
def test_short_chains_match_reference_and_separate_glue(rows, hidden, kv_heads):
    """hidden 4096 / 8192: the qkv and gate-up matvecs compute their activations from the previous accumulator (six
    launches per block), and the down projection makes its SwiGLU input itself (five); one more with grouped-query
    attention."""
    from rptc_b200 import ops
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    cfg = LlamaConfig(hidden=hidden, layers=4, heads=hidden // 128, kv_heads=kv_heads, ffn=1792, vocab=512, max_pos=16,
                      weight_scale=0.02 if hidden == 4096 else 0.014)
    T = 6
    model = RPTCLlama(cfg, rows=rows, seed=3)
    assert model._glueable() and model._mlp_glueable()
    gqa = 0 if kv_heads == hidden // 128 else 1
    g = torch.Generator(device="cuda").manual_seed(5)
    tokens = torch.randint(0, cfg.vocab, (rows, T), device="cuda", generator=g)
    ref = model.reference_logits(tokens)
    logits = {}
    # (launches per block, glue inside the matvecs, SwiGLU inside the down projection, q/k/v finish inside attention).
    # The chains with the glue in launches of their own fuse the attention front end for multi-head attention only;
    # the glued chains fuse it for grouped-query attention too (a later launch zeroes the qkv accumulator).
    variants = [(8 + gqa, False, False, True), (7 + gqa, False, True, True), (6, True, False, True), (5, True, True, True),
                (6, True, True, False)]
    for launches, glued, glued_mlp, fuse_attention in variants:
        model.glued, model.glued_mlp, model.fuse_attention = glued, glued_mlp, fuse_attention
        key = (launches, glued, glued_mlp, fuse_attention)
        for use_graph in (False, True):
            model.reset()
            model.graph = None
            if use_graph:
                model.capture(pdl=True)
            for t in range(T):
                model.ids.copy_(tokens[:, t].to(torch.int32))
                model.step()
                torch.cuda.synchronize()
                got = model.logits.float()
                err = (got - ref[:, t]).abs().max().item()
                # 4096-long dot products of fp16 activations: twice the slack of the small models above
                assert err <= 2e-2 * ref[:, t].abs().max().item(), (key, use_graph, t, err)
                logits[key, use_graph, t] = got.clone()
            assert model.launches_per_step == launches * cfg.layers + 4, key
            # the accumulators with an owner are handed back zeroed, whichever launch did the clearing
            model.graph = None
            ops.embed(model.embed, model.ids, model.h)        # any launch after the step: orders the check below
            torch.cuda.synchronize()
            assert not model.acc_qkv.any() and not model.acc_h.any(), key
            assert glued_mlp or not model.acc_gu.any()        # otherwise left to the next token's first launch
    model.fuse_attention = True
    for t in range(T):
        scale = ref[:, t].abs().max().item()
        for key in variants[1:]:
            # two fp16 pipelines whose partial sums meet in different orders (and, at two rows, in different kernels)
            assert (logits[key, True, t] - logits[variants[0], True, t]).abs().max().item() <= 1e-2 * scale


def test_next_token_kernel_matches_argmax():
    from rptc_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(2)
    logits = torch.randn((3, 32000), device="cuda", generator=g).half()
    logits[1, 777] = logits[1, 31999] = 9.0                       # a tie: the first maximum wins
    nxt = torch.zeros(3, dtype=torch.int64, device="cuda")
    ids = torch.zeros(3, dtype=torch.int32, device="cuda")
    pos = torch.tensor([4, 5, 6], dtype=torch.int32, device="cuda")
    mirror = torch.zeros(3, dtype=torch.int64).pin_memory()
    ops.next_token(logits, nxt, ids, pos, mirror)
    torch.cuda.synchronize()
    want = logits.float().argmax(dim=1)
    want[1] = 777
    assert torch.equal(nxt, want) and torch.equal(ids.long(), want) and pos.tolist() == [5, 6, 7]
    assert torch.equal(mirror, want.cpu())


def test_host_token_io_generates_the_same_tokens():
    """Token ids through pinned host memory (read by the first kernel, written by the last) against the
    device-resident feedback loop."""
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    cfg = LlamaConfig(hidden=512, layers=2, heads=4, kv_heads=4, ffn=1024, vocab=1024, max_pos=32, weight_scale=0.05)
    model = RPTCLlama(cfg, rows=1, seed=4)
    model.reset(torch.tensor([17]))
    model.capture()
    dev_tokens = []
    for _ in range(8):
        model.step()
        dev_tokens.append(int(model.next_ids.item()))
    host_in = torch.tensor([17], dtype=torch.int32).pin_memory()
    host_out = torch.zeros(1, dtype=torch.int64).pin_memory()
    model.bind_host_io(host_in, host_out)
    model.reset()
    model.capture()
    host_tokens = []
    for _ in range(8):
        model.step()
        torch.cuda.current_stream().synchronize()
        host_tokens.append(int(host_out[0]))
        host_in[0] = host_tokens[-1]
    assert host_tokens == dev_tokens
    with pytest.raises(ValueError):
        model.bind_host_io(torch.zeros(1, dtype=torch.int32), host_out)       # not pinned


def test_host_token_loop_with_a_launch_queued_ahead():
    """The mailbox loop (next step queued before its token is known) generates the device-resident loop's tokens."""
    from rptc_b200 import ops
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    cfg = LlamaConfig(hidden=512, layers=2, heads=4, kv_heads=4, ffn=1024, vocab=1024, max_pos=48, weight_scale=0.05)
    model = RPTCLlama(cfg, rows=2, seed=4)
    model.reset(torch.tensor([17, 400]))
    model.capture()
    dev_tokens = []
    for _ in range(12):
        model.step()
        dev_tokens.append(model.next_ids.tolist())
    loop = model.host_loop(timeout_ms=2000)
    model.reset()
    first = loop.run([17, 400], 5)
    rest = loop.run(first[-1], 7)                       # a second call continues the sequence numbers
    torch.cuda.synchronize()
    assert first + rest == dev_tokens
    assert model.pos.tolist() == [12, 12]
    ops.device_status()


def test_mailbox_wait_runs_out_and_reports():
    """Nobody posts the ids: the kernel gives up after its time limit, the stream drains, the status says so."""
    import time
    from rptc_b200 import RPTCError, ops
    table = torch.randn((64, 256), device="cuda").half()
    slots = torch.zeros(1, dtype=torch.int64).pin_memory()
    steps_done = torch.zeros(1, dtype=torch.int32, device="cuda")
    ids = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros((1, 256), dtype=torch.float16, device="cuda")
    t0 = time.perf_counter()
    ops.embed_mailbox(table, slots, steps_done, ids, out, timeout_ms=50)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    with pytest.raises(RPTCError):
        ops.device_status()
    ops.device_status()                                  # the report clears the word
    assert torch.equal(out[0], table[0])                 # it went on with the id it found
    slots[0] = (2 << 32) | 9                             # a posted entry is taken at once
    ops.embed_mailbox(table, slots, steps_done, ids, out, timeout_ms=50)
    torch.cuda.synchronize()
    ops.device_status()
    assert torch.equal(out[0], table[9]) and int(steps_done) == 2


@pytest.mark.parametrize("kv_heads", [2, 4])
def test_prefill_on_the_tensor_core_gemm_then_decode(kv_heads):
    """A 40-token prompt in one pass through the fused dequant-GEMM, then token-by-token decoding from the caches it
    filled: logits against the fp32 reference of the same network at every position that is checked."""
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    cfg = LlamaConfig(hidden=512, layers=2, heads=4, kv_heads=kv_heads, ffn=1024, vocab=1024, max_pos=64, weight_scale=0.05)
    rows, T, extra = 2, 40, 5
    model = RPTCLlama(cfg, rows=rows, seed=9)
    g = torch.Generator(device="cuda").manual_seed(13)
    tokens = torch.randint(0, cfg.vocab, (rows, T + extra), device="cuda", generator=g)
    ref = model.reference_logits(tokens)
    model.reset()
    got = model.prefill(tokens[:, :T]).float()
    torch.cuda.synchronize()
    err = (got - ref[:, T - 1]).abs().max().item()
    assert err <= 1.5e-2 * ref[:, T - 1].abs().max().item(), err
    assert model.pos.tolist() == [T] * rows
    assert torch.equal(model.ids.long(), got.argmax(dim=1))
    model.capture()
    for t in range(T, T + extra):                         # decode continues from the prefilled caches
        model.ids.copy_(tokens[:, t].to(torch.int32))
        model.step()
        torch.cuda.synchronize()
        err = (model.logits.float() - ref[:, t]).abs().max().item()
        assert err <= 1.5e-2 * ref[:, t].abs().max().item(), (t, err)


@pytest.mark.parametrize("kv_heads", [2, 4])
def test_decode_attention_beyond_one_chunk_of_positions(kv_heads):
    """Contexts of 300-560 positions: the attention kernel takes two and three chunks of 256 positions through its
    registers (online softmax across chunks), in both its forms (q/k/v finish fused in, or not)."""
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    cfg = LlamaConfig(hidden=512, layers=2, heads=4, kv_heads=kv_heads, ffn=1024, vocab=1024, max_pos=600, weight_scale=0.05)
    rows = 2
    model = RPTCLlama(cfg, rows=rows, seed=21)
    g = torch.Generator(device="cuda").manual_seed(23)
    for T in (300, 555):
        tokens = torch.randint(0, cfg.vocab, (rows, T + 4), device="cuda", generator=g)
        ref = model.reference_logits(tokens)
        model.reset()
        model.graph = None
        model.prefill(tokens[:, :T])
        model.capture()
        for t in range(T, T + 4):
            model.ids.copy_(tokens[:, t].to(torch.int32))
            model.step()
            torch.cuda.synchronize()
            err = (model.logits.float() - ref[:, t]).abs().max().item()
            assert err <= 1.5e-2 * ref[:, t].abs().max().item(), (T, t, err)


def test_a_step_beyond_the_cache_is_refused_on_the_host_and_skipped_on_the_device():
    """max_pos = 8.  The host counts the steps and refuses the ninth; when the host guard is bypassed the kernels
    themselves see the position, skip the cache write, raise the device status word, and a guard region behind the
    caches stays untouched.  Nothing faults: the access is skipped, not attempted."""
    from rptc_b200 import RPTCError, ops
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    # fused q/k/v finish + attention (multi-head and grouped-query), and the separate kernels
    for kv_heads, fuse_attention in ((4, True), (2, True), (2, False)):
        cfg = LlamaConfig(hidden=512, layers=2, heads=4, kv_heads=kv_heads, ffn=1024, vocab=512, max_pos=8, weight_scale=0.05)
        model = RPTCLlama(cfg, rows=1, seed=2)
        model.fuse_attention = fuse_attention
        # caches re-seated inside larger buffers whose tails are the guard regions
        guards = []
        for name in ("kcache", "vcache"):
            for i in range(cfg.layers):
                big = torch.full((1, cfg.max_pos + 4, kv_heads, cfg.head_dim), 7.0, dtype=torch.float16, device="cuda")
                getattr(model, name)[i] = big[:, : cfg.max_pos]
                guards.append(big)
        model.reset(torch.tensor([3]))
        for _ in range(cfg.max_pos):
            model.step()
        torch.cuda.synchronize()
        ops.device_status()                                   # eight steps fit
        with pytest.raises(RuntimeError, match="max_pos"):
            model.step()
        model.step_eager()                                    # around the host guard: position 8 reaches the kernels
        torch.cuda.synchronize()
        with pytest.raises(RPTCError) as err:
            ops.device_status()
        assert err.value.status == -10                        # RPTC_ERR_RANGE
        for big in guards:
            assert bool((big[:, cfg.max_pos:] == 7.0).all()), "a kernel wrote behind the cache"
        ops.device_status()                                   # the report cleared the word


def test_rope_cache_kernel_skips_a_position_outside_the_cache():
    from rptc_b200 import RPTCError, ops
    hq, hkv, d, max_pos = 4, 2, 128, 8
    qkv = torch.randn((1, (hq + 2 * hkv) * d), dtype=torch.float16, device="cuda")
    before = qkv.clone()
    big_k = torch.full((1, max_pos + 2, hkv, d), 7.0, dtype=torch.float16, device="cuda")
    big_v = big_k.clone()
    for bad in (8, -1, 2**31 - 1):
        pos = torch.tensor([bad], dtype=torch.int32, device="cuda")
        ops.rope_cache(qkv, pos, big_k[:, :max_pos], big_v[:, :max_pos], hq, hkv, d, 10000.0)
        torch.cuda.synchronize()
        with pytest.raises(RPTCError):
            ops.device_status()
        assert torch.equal(qkv, before) and bool((big_k == 7.0).all()) and bool((big_v == 7.0).all())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_two_devices_in_one_process():
    """The opt-in to large dynamic shared memory is per device: the kernels must work on the second device a process
    uses, not only on the first (plain local memory on each device, no peer operands)."""
    from rptc_b200 import Format, ops
    fmt = Format()
    m, n = 256, 4096
    results = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            g = torch.Generator(device=f"cuda:{dev}").manual_seed(5)
            codes = torch.randint(-2**31, 2**31 - 1, (m // 32, n // 64, 32, 4), dtype=torch.int32, device=f"cuda:{dev}", generator=g)
            lut = torch.randn(512, dtype=torch.float16, device=f"cuda:{dev}", generator=g)
            x = torch.eye(n, dtype=torch.float16, device=f"cuda:{dev}")[:8]
            y8 = ops.gemv(codes, lut, x, m, n, fmt)
            y1 = ops.gemv(codes, lut, x[:1], m, n, fmt)
            dense = ops.decompress(codes, lut, m, n, fmt)
            yg = ops.gemm(codes[: 128 // 32], lut, torch.eye(n, dtype=torch.float16, device=f"cuda:{dev}")[:256], 128, n, fmt)
            torch.cuda.synchronize()
            ops.device_status()
            assert torch.equal(y8, dense.t()[:8]) and torch.equal(y1, dense.t()[:1]) and torch.equal(yg, dense[:128].t()[:256])
            results.append(dense.cpu())
    assert torch.equal(results[0], results[1])


@pytest.mark.parametrize("kv_heads", [4, 2])
def test_decode_sixteen_rows_at_once(kv_heads):
    """Decode batch 16 (the reference's kernels take one activation vector only, inference.cu:291 `V == 1`): sixteen
    sequences step together, every fused matvec runs as two launches of eight rows; logits of every row against the fp32
    forward, eager and from the captured graph."""
    from rptc_b200 import ops
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    cfg = LlamaConfig(hidden=1024, layers=2, heads=8, kv_heads=kv_heads * 2, ffn=2816, vocab=1024, max_pos=32, weight_scale=0.05)
    rows, T = 16, 6
    model = RPTCLlama(cfg, rows=rows, seed=11)
    g = torch.Generator(device="cuda").manual_seed(3)
    tokens = torch.randint(0, cfg.vocab, (rows, T), device="cuda", generator=g)
    ref = model.reference_logits(tokens)
    for use_graph in (False, True):
        model.reset()
        model.graph = None
        if use_graph:
            model.capture(pdl=True)
        for t in range(T):
            model.ids.copy_(tokens[:, t].to(torch.int32))
            model.step()
            torch.cuda.synchronize()
            err = (model.logits.float() - ref[:, t]).abs().amax(dim=1) / ref[:, t].abs().amax(dim=1)
            assert float(err.max()) <= 1e-2, (use_graph, t, err.tolist())
        assert model.pos.tolist() == [T] * rows
    ops.device_status()


def test_fused_matvec_sixteen_rows_matches_two_calls_of_eight():
    from rptc_b200 import Format, ops
    fmt = Format()
    m, n = 1024, 4096
    g = torch.Generator(device="cuda").manual_seed(8)
    codes = torch.randint(-2**31, 2**31 - 1, ops.codes_shape(m, n, 2, fmt.layout), dtype=torch.int32, device="cuda", generator=g)
    lut = torch.randn(512, dtype=torch.float16, device="cuda", generator=g)
    x = torch.eye(n, dtype=torch.float16, device="cuda")[100:116]          # sixteen unit vectors: exact
    y = ops.gemv(codes, lut, x, m, n, fmt)
    dense = ops.decompress(codes, lut, m, n, fmt)
    assert torch.equal(y, dense.t()[100:116])
    y13 = ops.gemv(codes, lut, x[:13], m, n, fmt)                           # 8 + 4 + 1
    assert torch.equal(y13, dense.t()[100:113])
