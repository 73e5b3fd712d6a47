"""A Llama-architecture decoder over RPTC-quantised linears: the decode engine the benchmark times.

Every linear of every block (fused qkv, o, fused gate-up, down) is an RPTCLinear over packed
codes; embeddings, norms and the output head stay fp16 (the reference quantises only
self_attn.*_proj and mlp.*_proj, quantize_hf.py:189).  One decode step is a fixed sequence of
kernel launches on one stream, captured once in a CUDA graph and replayed per token; with
programmatic dependent launch the table set-up and first weight fetches of each fused
dequant-GEMV overlap the small kernel in front of it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import ops
from ._lib import CODE_HASH, LAYOUT_TILED, Format, lib
from .linear import RPTCLinear, hadamard_block


@dataclass
class LlamaConfig:
    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 32
    ffn: int = 11008
    vocab: int = 32000
    head_dim: int = 128
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_pos: int = 512
    weight_scale: float = 0.02

    @classmethod
    def llama2_7b(cls, **kw):
        return cls(**kw)

    @classmethod
    def llama2_70b(cls, **kw):
        return cls(hidden=8192, layers=80, heads=64, kv_heads=8, ffn=28672, **kw)

    def quantised_weights(self) -> int:
        q = self.heads * self.head_dim
        kv = self.kv_heads * self.head_dim
        per_layer = self.hidden * (q + 2 * kv) + q * self.hidden + 3 * self.hidden * self.ffn
        return per_layer * self.layers


class Block:
    """One decoder block's weights.  With tensor parallelism (tp > 1) the block holds this rank's
    shard: qkv and gate-up are split by output rows (heads / FFN channels), o and down by input
    columns, and the Hadamard blocks are sized so that no block straddles a shard boundary."""

    def __init__(self, cfg: LlamaConfig, fmt: Format, seed: int, device, incoherent: bool, tp: int = 1, norm_seed: int | None = None):
        q, kv, ffn = cfg.heads * cfg.head_dim // tp, cfg.kv_heads * cfg.head_dim // tp, cfg.ffn // tp
        mk = lambda i, o, s: RPTCLinear.random(i, o, fmt, cfg.weight_scale, seed * 16 + s, device, incoherent)
        self.qkv = mk(cfg.hidden, q + 2 * kv, 0)
        # per-head output transform: lets one kernel finish q, k, v of a head and attend
        self.qkv.block_out = cfg.head_dim if cfg.head_dim == 128 else hadamard_block(math.gcd(q, kv))
        self.o = mk(q, cfg.hidden, 1)
        self.o.block_in = min(self.o.block_in, cfg.head_dim)      # one Hadamard block per head: fuses into the attention kernel
        self.gate_up = mk(cfg.hidden, 2 * ffn, 2)
        # gate and up are transformed separately, so that the fused SwiGLU kernel can own matching blocks of both
        self.gate_up.block_out = min(hadamard_block(ffn), 256)        # at most 256: the SwiGLU middle stays warp-local
        self.down = mk(ffn, cfg.hidden, 3)
        self.down.block_in = self.gate_up.block_out
        g = torch.Generator(device=device).manual_seed((seed if norm_seed is None else norm_seed) * 16 + 9)   # replicated
        self.norm1 = (1.0 + 0.1 * torch.randn(cfg.hidden, generator=g, device=device)).to(torch.float16)
        self.norm2 = (1.0 + 0.1 * torch.randn(cfg.hidden, generator=g, device=device)).to(torch.float16)

    def linears(self):
        return [self.qkv, self.o, self.gate_up, self.down]


class RPTCLlama:
    """Random-init Llama-shape model with all block linears RPTC-quantised; batch-`rows` decode."""

    def __init__(self, cfg: LlamaConfig, fmt: Format | None = None, rows: int = 1, seed: int = 0, device="cuda",
                 incoherent: bool = True, tp_world: int = 1, tp_rank: int = 0, tp_group=None, peer_allreduce: bool = False):
        """tp_world > 1: this object is rank `tp_rank`'s shard of a tensor-parallel model; the partial
        outputs of the row-parallel layers (o, down) are summed over `tp_group` with an NCCL all-reduce.
        Embedding, norms and output head are replicated (same seed on every rank)."""
        self.cfg, self.rows, self.device = cfg, rows, torch.device(device)
        self.tp_world, self.tp_rank, self.tp_group = tp_world, tp_rank, tp_group
        if cfg.heads % tp_world or cfg.kv_heads % tp_world or cfg.ffn % (tp_world * 64):
            raise ValueError("heads, kv_heads and ffn/64 must be divisible by the tensor-parallel degree")
        self.fmt = fmt or Format(CODE_HASH, 2, 16, 8, LAYOUT_TILED)
        self.blocks = [Block(cfg, self.fmt, (seed * 64 + tp_rank) * 1000 + i + 1, device, incoherent, tp_world,
                             norm_seed=seed * 64000 + i + 1) for i in range(cfg.layers)]
        g = torch.Generator(device=device).manual_seed(seed * 1000 + 999)
        self.embed = (torch.randn(cfg.vocab, cfg.hidden, generator=g, device=device) * 0.02).to(torch.float16)
        self.head = (torch.randn(cfg.vocab, cfg.hidden, generator=g, device=device) * 0.02).to(torch.float16)
        self.norm_f = (1.0 + 0.1 * torch.randn(cfg.hidden, generator=g, device=device)).to(torch.float16)
        self.heads_l, self.kv_heads_l, self.ffn_l = cfg.heads // tp_world, cfg.kv_heads // tp_world, cfg.ffn // tp_world
        q, kv = self.heads_l * cfg.head_dim, self.kv_heads_l * cfg.head_dim
        f16 = dict(dtype=torch.float16, device=device)
        self.kcache = [torch.zeros((rows, cfg.max_pos, self.kv_heads_l, cfg.head_dim), **f16) for _ in range(cfg.layers)]
        self.vcache = [torch.zeros((rows, cfg.max_pos, self.kv_heads_l, cfg.head_dim), **f16) for _ in range(cfg.layers)]
        # step workspace (fixed addresses, so that the step can live in a CUDA graph)
        self.ids = torch.zeros(rows, dtype=torch.int32, device=device)
        self.pos = torch.zeros(rows, dtype=torch.int32, device=device)
        self.h = torch.zeros((rows, cfg.hidden), **f16)
        self.xn = torch.zeros((rows, cfg.hidden), **f16)
        self.xt = torch.zeros((rows, max(cfg.hidden, q)), **f16)
        self.qkv_out = torch.zeros((rows, q + 2 * kv), **f16)
        self.attn = torch.zeros((rows, q), **f16)
        self.mlp = torch.zeros((rows, self.ffn_l), **f16)
        self.partial = torch.zeros((rows, cfg.hidden), **f16)
        self.logits = torch.zeros((rows, cfg.vocab), **f16)
        self.next_ids = torch.zeros(rows, dtype=torch.int64, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        # acc_qkv and acc_h share one allocation: with grouped-query attention the fused attention kernel cannot zero the
        # k and v columns it reads (several q heads read them), so the launch that zeroes acc_h zeroes acc_qkv with it
        self._acc_pool2 = torch.zeros(rows * (q + 2 * kv + cfg.hidden), **f32)
        self.acc_qkv = self._acc_pool2[: rows * (q + 2 * kv)].view(rows, q + 2 * kv)
        self.acc_h = self._acc_pool2[rows * (q + 2 * kv):].view(rows, cfg.hidden)
        # second residual stream and accumulator of the shortest chain, whose matvecs compute their own inputs; the
        # accumulators that a later launch zeroes (acc_o, acc_gu) share one allocation so that one range covers both
        self.h2 = torch.zeros((rows, cfg.hidden), **f16)
        self._acc_pool = torch.zeros(rows * (cfg.hidden + 2 * self.ffn_l), **f32)
        self.acc_o = self._acc_pool[: rows * cfg.hidden].view(rows, cfg.hidden)
        self.acc_gu = self._acc_pool[rows * cfg.hidden:].view(rows, 2 * self.ffn_l)
        self.acc_gu2 = torch.zeros_like(self.acc_gu)     # second gate-up accumulator of the chains that alternate two
        self.peer = None
        if tp_world > 1 and peer_allreduce and incoherent:
            # the fused transform + all-reduce + residual kernel over NVLink peer memory instead of NCCL
            from .tp import PeerAllReduce
            self.peer = PeerAllReduce(rows, cfg.hidden, self.blocks[0].o.block_out, tp_rank, tp_world, tp_group)
        self.glued = True           # False keeps the glue in launches of its own (the 8-launch chain)
        self.fused_tp = True        # False: the 15-launch chain under tensor parallelism
        self.glued_mlp = True       # False: SwiGLU in a launch of its own inside the short chain
        self.glued_tp = True        # False: RMSNorm + input transform of the tensor-parallel chain in launches of their own
        self.fuse_attention = True  # False: q/k/v finish + RoPE + KV append in a launch of their own, in front of attention
        self.host_ids: torch.Tensor | None = None      # see bind_host_io
        self.host_next: torch.Tensor | None = None
        self.mailbox = None                            # see bind_mailbox
        self.graph: torch.cuda.CUDAGraph | None = None
        self.launches_per_step = 0
        self._pos_hi = 0            # host-side upper bound of the positions on the device (see step)

    # -- one token for every row ---------------------------------------------------------------------
    def _fusable(self) -> bool:
        """The fused chain (8 launches per block) needs incoherent layers, no tensor parallelism, and a
        hidden size that is a single Hadamard block (or two of 4096)."""
        n = self.cfg.hidden
        return (self.tp_world == 1 and self.blocks[0].qkv.incoherent and n & (n - 1) == 0 and 256 <= n <= 8192
                and self.cfg.head_dim == 128)

    def _glueable(self) -> bool:
        """The short chain (5 launches per block with multi-head attention, 6 with grouped-query attention)
        additionally needs hidden 4096 or 8192 (one or two 4096-point blocks, eight values a thread of the 512-thread
        matvec CTA each) and at most two rows."""
        b = self.blocks[0]
        return (self._fusable() and self.cfg.hidden in (4096, 8192) and self.rows <= 2 and b.qkv.block_out >= 128
                and self.fmt.layout == LAYOUT_TILED and self.fmt.K in (2, 4) and self.glued)

    def _mlp_glueable(self) -> bool:
        """The down projection can make its own activations (five launches per block) when the MLP width is a whole
        number of 256-column blocks and both transforms around the SwiGLU use blocks of at most 256."""
        b = self.blocks[0]
        return (self.glued_mlp and self.ffn_l % 256 == 0 and b.down.block_in <= 256 and b.down.block_in == b.gate_up.block_out)

    def _fusable_tp(self) -> bool:
        """The tensor-parallel short chain (11 launches per block with the peer all-reduce): incoherent layers, hidden a
        power of two up to 8192 (one or two 4096-point Hadamard blocks), 128-wide heads."""
        n = self.cfg.hidden
        return (self.tp_world > 1 and self.blocks[0].qkv.incoherent and n & (n - 1) == 0 and 256 <= n <= 8192
                and self.cfg.head_dim == 128 and self.blocks[0].qkv.block_out >= 128 and self.fused_tp)

    def _extra_launches(self) -> int:
        """Launches beyond one per matvec: a fused matvec takes up to eight activation rows per launch (8 + 8 at sixteen
        rows, 4 + 1 at five), and so does the output head."""
        q, r = divmod(self.rows, 8)
        per_matvec = q + bin(r).count("1") - 1
        return 4 * per_matvec * len(self.blocks) + (self.rows - 1) // 8

    def step_eager(self) -> None:
        if self._glueable():
            self._step_glued()
        elif self._fusable_tp():
            self._step_fused_tp()
        elif self._fusable():
            self._step_fused()
        else:
            self._step_unfused()

    def _embed_ids(self) -> None:
        if self.mailbox is not None:
            slots_in, _, steps_done, timeout_ms = self.mailbox
            ops.embed_mailbox(self.embed, slots_in, steps_done, self.ids, self.h, timeout_ms)
        else:
            ops.embed(self.embed, self.ids if self.host_ids is None else self.host_ids, self.h)

    def _next_token(self) -> None:
        if self.mailbox is not None:
            ops.next_token(self.logits, self.next_ids, None, self.pos, self.mailbox[1], self.mailbox[2])
        else:
            ops.next_token(self.logits, self.next_ids, self.ids, self.pos, self.host_next)

    def _step_fused(self) -> None:
        cfg = self.cfg
        q_dim = self.heads_l * cfg.head_dim
        self._embed_ids()
        b0 = self.blocks[0]
        xt = self.xt[:, : cfg.hidden]
        ops.finish_norm_hadamard(None, None, 1.0, self.h, b0.norm1, cfg.rms_eps, b0.qkv.signs_in, True, xt)
        n_launch = 2
        mlp_glued = (self._mlp_glueable() and self.rows <= 2 and len(self.blocks) % 2 == 0 and self.fmt.layout == LAYOUT_TILED
                     and self.fmt.K in (2, 4))
        for i, b in enumerate(self.blocks):
            b.qkv.matvec_acc(xt, self.acc_qkv)
            if self.fuse_attention and self.heads_l == self.kv_heads_l and b.qkv.block_out == 128:
                ops.qkv_attn_decode(self.acc_qkv, b.qkv.signs_out, b.qkv.scale, self.pos, self.kcache[i], self.vcache[i], self.attn,
                                    self.heads_l, self.kv_heads_l, cfg.rope_theta, b.o.signs_in)
                n_launch -= 1
            else:
                ops.qkv_finish(self.acc_qkv, b.qkv.signs_out, b.qkv.scale, self.qkv_out, self.kcache[i], self.vcache[i], self.pos,
                               self.heads_l, self.kv_heads_l, b.qkv.block_out, cfg.rope_theta)
                ops.attn_decode(self.qkv_out, self.pos, self.kcache[i], self.vcache[i], self.attn, self.heads_l, self.kv_heads_l,
                                cfg.head_dim, signs_in=b.o.signs_in)
            b.o.matvec_acc(self.attn, self.acc_h)
            ops.finish_norm_hadamard(self.acc_h, b.o.signs_out, b.o.scale, self.h, b.norm2, cfg.rms_eps, b.gate_up.signs_in, True, xt)
            if mlp_glued:
                # the down projection makes its SwiGLU input itself; two gate-up accumulators alternate from block to
                # block and each down projection zeroes the one the block before it used
                gu, other = (self.acc_gu, self.acc_gu2) if i % 2 == 0 else (self.acc_gu2, self.acc_gu)
                b.gate_up.matvec_acc(xt, gu)
                ops.gemv_swiglu_input(b.down.codes, b.down.lut, self.acc_h, cfg.hidden, self.ffn_l, self.fmt, self.rows, gu,
                                      b.gate_up.signs_out, b.gate_up.scale, b.down.signs_in, b.down.block_in, clear=other,
                                      carry_in=b.down.carry_in)
                n_launch -= 1
            else:
                b.gate_up.matvec_acc(xt, self.acc_gu)
                ops.swiglu_hadamard(self.acc_gu, self.mlp, b.gate_up.signs_out, b.down.signs_in, self.ffn_l, b.down.block_in,
                                    b.gate_up.scale, 1.0, clear=True)
                b.down.matvec_acc(self.mlp, self.acc_h)
            if i + 1 < len(self.blocks):
                nb = self.blocks[i + 1]
                ops.finish_norm_hadamard(self.acc_h, b.down.signs_out, b.down.scale, self.h, nb.norm1, cfg.rms_eps,
                                         nb.qkv.signs_in, True, xt)
            else:
                ops.finish_norm_hadamard(self.acc_h, b.down.signs_out, b.down.scale, self.h, self.norm_f, cfg.rms_eps, None, False,
                                         self.xn)
            n_launch += 9
        ops.dense_gemv(self.head, self.xn, out=self.logits)
        self._next_token()
        self.launches_per_step = n_launch + 2 + self._extra_launches()

    def _step_glued(self) -> None:
        """qkv matvec -> attention -> o matvec -> gate-up matvec -> SwiGLU -> down matvec.  The two matvecs that
        follow a row-parallel layer compute their activations (residual update, RMSNorm, input transform) from
        that layer's accumulator themselves.  The residual stream alternates between h and h2; an accumulator
        that every CTA of a launch reads is zeroed by a later launch (`clear`)."""
        cfg, r = self.cfg, self.rows
        self._embed_ids()
        mlp_glued = self._mlp_glueable()
        mha = self.fuse_attention and self.blocks[0].qkv.block_out == 128 and cfg.head_dim == 128
        gqa = self.heads_l != self.kv_heads_l
        # the launch that opens a block zeroes what the block before it left: acc_o always, acc_gu too when the down
        # projection reads it in every CTA
        stale = self._acc_pool if mlp_glued else self.acc_o
        for i, b in enumerate(self.blocks):
            prev = self.blocks[i - 1].down if i else None
            ops.gemv_norm_input(b.qkv.codes, b.qkv.lut, self.acc_qkv, b.qkv.out_features, cfg.hidden, self.fmt, r,
                                self.acc_h if prev else None, prev.signs_out if prev else None, prev.scale if prev else 1.0,
                                self.h, self.h2, b.norm1, cfg.rms_eps, b.qkv.signs_in, clear=stale)
            if mha:
                ops.qkv_attn_decode(self.acc_qkv, b.qkv.signs_out, b.qkv.scale, self.pos, self.kcache[i], self.vcache[i], self.attn,
                                    self.heads_l, self.kv_heads_l, cfg.rope_theta, b.o.signs_in)
            else:
                ops.qkv_finish(self.acc_qkv, b.qkv.signs_out, b.qkv.scale, self.qkv_out, self.kcache[i], self.vcache[i], self.pos,
                               self.heads_l, self.kv_heads_l, b.qkv.block_out, cfg.rope_theta)
                ops.attn_decode(self.qkv_out, self.pos, self.kcache[i], self.vcache[i], self.attn, self.heads_l, self.kv_heads_l,
                                cfg.head_dim, signs_in=b.o.signs_in)
            b.o.matvec_acc(self.attn, self.acc_o)
            # acc_h was consumed by this block's first launch; with grouped-query attention acc_qkv is zeroed here too
            stale_h = self._acc_pool2 if (mha and gqa) else (self.acc_h if i else None)
            ops.gemv_norm_input(b.gate_up.codes, b.gate_up.lut, self.acc_gu, b.gate_up.out_features, cfg.hidden, self.fmt, r,
                                self.acc_o, b.o.signs_out, b.o.scale, self.h2, self.h, b.norm2, cfg.rms_eps, b.gate_up.signs_in,
                                clear=stale_h)
            if mlp_glued:
                ops.gemv_swiglu_input(b.down.codes, b.down.lut, self.acc_h, cfg.hidden, self.ffn_l, self.fmt, r, self.acc_gu,
                                      b.gate_up.signs_out, b.gate_up.scale, b.down.signs_in, b.down.block_in,
                                      carry_in=b.down.carry_in)
            else:
                ops.swiglu_hadamard(self.acc_gu, self.mlp, b.gate_up.signs_out, b.down.signs_in, self.ffn_l, b.down.block_in,
                                    b.gate_up.scale, 1.0, clear=True)
                b.down.matvec_acc(self.mlp, self.acc_h)
        last = self.blocks[-1].down
        ops.finish_norm_hadamard(self.acc_h, last.signs_out, last.scale, self.h, self.norm_f, cfg.rms_eps, None, False, self.xn)
        ops.dense_gemv(self.head, self.xn, out=self.logits)
        self._next_token()
        self.launches_per_step = ((5 if mlp_glued else 6) + (0 if mha else 1)) * len(self.blocks) + 4

    def _step_fused_tp(self) -> None:
        """Tensor-parallel decode step with the glue fused as far as the all-reduce allows: RMSNorm + input transform in
        one kernel, q/k/v finish + RoPE + KV append in one, the output projection's input transform inside attention,
        the gated-MLP middle in one; the row-parallel layers end in the all-reduce (+ transform + residual)."""
        cfg = self.cfg
        xt = self.xt[:, : cfg.hidden]
        self._embed_ids()
        b0 = self.blocks[0]
        per_reduce = 1 if self.peer is not None else 3
        native = self.rows <= 2 and self.fmt.layout == LAYOUT_TILED and self.fmt.K in (2, 4)
        mlp_glued = self._mlp_glueable() and native and len(self.blocks) % 2 == 0
        # RMSNorm + input transform inside the matvec that consumes them (the all-reduce has already updated h)
        norm_glued = self.glued_tp and native and cfg.hidden in (4096, 8192)

        def normed_matvec(lin, w_norm, acc, clear=None):
            ops.gemv_norm_input(lin.codes, lin.lut, acc, lin.out_features, cfg.hidden, self.fmt, self.rows, None, None, 1.0,
                                self.h, self.h2, w_norm, cfg.rms_eps, lin.signs_in, clear=clear, carry_in=lin.carry_in)

        if norm_glued:
            return self._step_fused_tp_glued(normed_matvec, mlp_glued, per_reduce)
        ops.finish_norm_hadamard(None, None, 1.0, self.h, b0.norm1, cfg.rms_eps, b0.qkv.signs_in, True, xt)
        for i, b in enumerate(self.blocks):
            b.qkv.matvec_acc(xt, self.acc_qkv)
            ops.qkv_finish(self.acc_qkv, b.qkv.signs_out, b.qkv.scale, self.qkv_out, self.kcache[i], self.vcache[i], self.pos,
                           self.heads_l, self.kv_heads_l, b.qkv.block_out, cfg.rope_theta)
            ops.attn_decode(self.qkv_out, self.pos, self.kcache[i], self.vcache[i], self.attn, self.heads_l, self.kv_heads_l,
                            cfg.head_dim, signs_in=b.o.signs_in)
            b.o.matvec_acc(self.attn, self.acc_h)
            self._finish_row_parallel(b.o)
            ops.finish_norm_hadamard(None, None, 1.0, self.h, b.norm2, cfg.rms_eps, b.gate_up.signs_in, True, xt)
            if mlp_glued:
                # The down projection makes its SwiGLU input from the gate-up accumulator in every CTA that needs a
                # piece of it, so nobody owns the clearing: two accumulators alternate from block to block and each
                # down projection zeroes the one the block before it used.
                gu, other = (self.acc_gu, self.acc_gu2) if i % 2 == 0 else (self.acc_gu2, self.acc_gu)
                b.gate_up.matvec_acc(xt, gu)
                ops.gemv_swiglu_input(b.down.codes, b.down.lut, self.acc_h, cfg.hidden, self.ffn_l, self.fmt, self.rows, gu,
                                      b.gate_up.signs_out, b.gate_up.scale, b.down.signs_in, b.down.block_in, clear=other,
                                      carry_in=b.down.carry_in)
            else:
                b.gate_up.matvec_acc(xt, self.acc_gu)
                ops.swiglu_hadamard(self.acc_gu, self.mlp, b.gate_up.signs_out, b.down.signs_in, self.ffn_l, b.down.block_in,
                                    b.gate_up.scale, 1.0, clear=True)
                b.down.matvec_acc(self.mlp, self.acc_h)
            self._finish_row_parallel(b.down)
            if i + 1 < len(self.blocks):
                nb = self.blocks[i + 1]
                ops.finish_norm_hadamard(None, None, 1.0, self.h, nb.norm1, cfg.rms_eps, nb.qkv.signs_in, True, xt)
            else:
                ops.finish_norm_hadamard(None, None, 1.0, self.h, self.norm_f, cfg.rms_eps, None, False, self.xn)
        ops.dense_gemv(self.head, self.xn, out=self.logits)
        self._next_token()
        self.launches_per_step = ((8 if mlp_glued else 9) + 2 * per_reduce) * len(self.blocks) + 4 + self._extra_launches()

    def _step_fused_tp_glued(self, normed_matvec, mlp_glued: bool, per_reduce: int) -> None:
        """The tensor-parallel chain with the norms inside the matvecs: qkv* -> attention (q/k/v finish inside or in
        front) -> o -> all-reduce -> gate-up* -> down (SwiGLU inside or in front) -> all-reduce."""
        cfg = self.cfg
        fused_attn = self.fuse_attention and self.blocks[0].qkv.block_out == 128 and cfg.head_dim == 128
        # grouped-query attention: the fused attention kernel leaves acc_qkv as it is and the gate-up launch zeroes it
        stale_qkv = self.acc_qkv if (fused_attn and self.heads_l != self.kv_heads_l) else None
        for i, b in enumerate(self.blocks):
            normed_matvec(b.qkv, b.norm1, self.acc_qkv)
            if fused_attn:
                ops.qkv_attn_decode(self.acc_qkv, b.qkv.signs_out, b.qkv.scale, self.pos, self.kcache[i], self.vcache[i], self.attn,
                                    self.heads_l, self.kv_heads_l, cfg.rope_theta, b.o.signs_in)
            else:
                ops.qkv_finish(self.acc_qkv, b.qkv.signs_out, b.qkv.scale, self.qkv_out, self.kcache[i], self.vcache[i], self.pos,
                               self.heads_l, self.kv_heads_l, b.qkv.block_out, cfg.rope_theta)
                ops.attn_decode(self.qkv_out, self.pos, self.kcache[i], self.vcache[i], self.attn, self.heads_l, self.kv_heads_l,
                                cfg.head_dim, signs_in=b.o.signs_in)
            b.o.matvec_acc(self.attn, self.acc_h)
            self._finish_row_parallel(b.o)
            if mlp_glued:
                gu, other = (self.acc_gu, self.acc_gu2) if i % 2 == 0 else (self.acc_gu2, self.acc_gu)
                normed_matvec(b.gate_up, b.norm2, gu, clear=stale_qkv)
                ops.gemv_swiglu_input(b.down.codes, b.down.lut, self.acc_h, cfg.hidden, self.ffn_l, self.fmt, self.rows, gu,
                                      b.gate_up.signs_out, b.gate_up.scale, b.down.signs_in, b.down.block_in, clear=other,
                                      carry_in=b.down.carry_in)
            else:
                normed_matvec(b.gate_up, b.norm2, self.acc_gu, clear=stale_qkv)
                ops.swiglu_hadamard(self.acc_gu, self.mlp, b.gate_up.signs_out, b.down.signs_in, self.ffn_l, b.down.block_in,
                                    b.gate_up.scale, 1.0, clear=True)
                b.down.matvec_acc(self.mlp, self.acc_h)
            self._finish_row_parallel(b.down)
        ops.finish_norm_hadamard(None, None, 1.0, self.h, self.norm_f, cfg.rms_eps, None, False, self.xn)
        ops.dense_gemv(self.head, self.xn, out=self.logits)
        self._next_token()
        self.launches_per_step = ((6 if mlp_glued else 7) - (1 if fused_attn else 0) + 2 * per_reduce) * len(self.blocks) + 4

    def _step_unfused(self) -> None:
        cfg, r = self.cfg, self.rows
        n_launch = 0
        self._embed_ids()
        n_launch += 1
        for i, b in enumerate(self.blocks):
            ops.rmsnorm(self.h, b.norm1, self.xn, cfg.rms_eps)
            xt = b.qkv.transform_in(self.xn, out=self.xt[:, : cfg.hidden])
            b.qkv.matvec_acc(xt, self.acc_qkv)
            b.qkv.finish(self.acc_qkv, out=self.qkv_out)
            ops.rope_cache(self.qkv_out, self.pos, self.kcache[i], self.vcache[i], self.heads_l, self.kv_heads_l, cfg.head_dim,
                           cfg.rope_theta)
            ops.attn_decode(self.qkv_out, self.pos, self.kcache[i], self.vcache[i], self.attn, self.heads_l, self.kv_heads_l,
                            cfg.head_dim)
            xt = b.o.transform_in(self.attn, out=self.xt[:, : self.attn.shape[1]])
            b.o.matvec_acc(xt, self.acc_h)
            self._finish_row_parallel(b.o)
            ops.rmsnorm(self.h, b.norm2, self.xn, cfg.rms_eps)
            xt = b.gate_up.transform_in(self.xn, out=self.xt[:, : cfg.hidden])
            b.gate_up.matvec_acc(xt, self.acc_gu)
            if b.gate_up.incoherent:
                ops.swiglu_hadamard(self.acc_gu, self.mlp, b.gate_up.signs_out, b.down.signs_in, self.ffn_l, b.down.block_in,
                                    b.gate_up.scale, 1.0, clear=True)
            else:
                gu = b.gate_up.finish(self.acc_gu)
                torch.mul(torch.nn.functional.silu(gu[:, : self.ffn_l]), gu[:, self.ffn_l:], out=self.mlp)
            n_launch += 15
            b.down.matvec_acc(self.mlp, self.acc_h)
            self._finish_row_parallel(b.down)
        ops.rmsnorm(self.h, self.norm_f, self.xn, cfg.rms_eps)
        ops.dense_gemv(self.head, self.xn, out=self.logits)
        self._next_token()
        self.launches_per_step = n_launch + 3 + self._extra_launches()

    def _finish_row_parallel(self, lin: RPTCLinear) -> None:
        """h += (sum over tensor-parallel ranks of) this rank's partial output of a row-parallel layer."""
        if self.tp_world == 1:
            lin.finish(self.acc_h, out=self.h, residual=self.h)
            return
        if self.peer is not None:
            self.peer.finish(lin, self.acc_h, self.h)
            return
        import torch.distributed as dist
        lin.finish(self.acc_h, out=self.partial)
        dist.all_reduce(self.partial, group=self.tp_group)
        self.h.add_(self.partial)

    def bind_host_io(self, host_ids: torch.Tensor | None, host_next: torch.Tensor | None) -> None:
        """Token ids in and out through pinned host memory without copies of their own: the step's first kernel reads
        `host_ids` (int32 [rows]) over PCIe, its last kernel writes the chosen ids to `host_next` (int64 [rows]); the host
        sees them once the stream is synchronised.  Call before `capture`; None restores device-resident feedback."""
        for t, dt in ((host_ids, torch.int32), (host_next, torch.int64)):
            if t is not None and (not t.is_pinned() or t.dtype != dt or t.numel() != self.rows):
                raise ValueError("host buffers must be pinned, int32 ids / int64 next ids, one element per row")
        self.host_ids, self.host_next = host_ids, host_next
        self.graph = None

    def bind_mailbox(self, timeout_ms: int = 2000):
        """Token ids through a mailbox in pinned host memory (see HostTokenLoop): the step's first kernel waits, for at
        most `timeout_ms`, until the host has posted the ids of this step.  Returns (slots_in, slots_out), pinned
        int64 [rows] holding (sequence << 32) | id.  Call before `capture`."""
        slots_in = torch.zeros(self.rows, dtype=torch.int64).pin_memory()
        slots_out = torch.zeros(self.rows, dtype=torch.int64).pin_memory()
        steps_done = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.host_ids = self.host_next = None
        self.mailbox = (slots_in, slots_out, steps_done, timeout_ms)
        self.graph = None
        return slots_in, slots_out

    def capture(self, pdl: bool = True) -> None:
        """Captures one decode step into a CUDA graph (after a warm-up step that is then undone)."""
        # Programmatic dependent launch is kept off when NCCL kernels sit in the same graph; the peer all-reduce is one
        # of this library's kernels and waits for the grid in front like the others.
        lib().rptc_set_pdl(1 if (pdl and (self.tp_world == 1 or self.peer is not None)) else 0)
        ids0, pos0 = self.ids.clone(), self.pos.clone()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            mailbox, self.mailbox = self.mailbox, None        # the warm-up step must not wait for a host that is here
            self.step_eager()
            self.mailbox = mailbox
            self.ids.copy_(ids0)
            self.pos.copy_(pos0)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=s):
                self.step_eager()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.ids.copy_(ids0)
        self.pos.copy_(pos0)
        lib().rptc_set_pdl(0)

    def host_loop(self, timeout_ms: int = 2000) -> "HostTokenLoop":
        return HostTokenLoop(self, timeout_ms)

    def sync_positions(self) -> None:
        """Re-reads the device-side positions after they were edited directly (`model.pos.copy_(...)`)."""
        self._pos_hi = int(self.pos.max().item())

    def _claim_positions(self, n_steps: int) -> None:
        """The positions live on the device and advance with every replay of the captured step; the host keeps an upper
        bound and refuses a step that has no row left in the KV caches (the kernels would skip the access and raise the
        device status word, but by then the token is lost)."""
        if self._pos_hi + n_steps > self.cfg.max_pos:
            raise RuntimeError(f"decode step at position {self._pos_hi + n_steps - 1} but the KV caches hold max_pos = "
                               f"{self.cfg.max_pos} positions")
        self._pos_hi += n_steps

    def step(self) -> None:
        self._claim_positions(1)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step_eager()

    def reset(self, ids: torch.Tensor | None = None) -> None:
        self.pos.zero_()
        self._pos_hi = 0
        self._acc_pool.zero_()      # the short chain leaves acc_o / acc_gu to the next token's first launch
        self.acc_gu2.zero_()
        if ids is not None:
            self.ids.copy_(ids.to(torch.int32))

    def bytes_per_token(self, context: int) -> dict:
        cfg = self.cfg
        packed = cfg.quantised_weights() * self.fmt.K // 8 // self.tp_world
        head = cfg.vocab * cfg.hidden * 2
        kv = 2 * cfg.layers * context * self.kv_heads_l * cfg.head_dim * 2
        return {"packed": packed, "head": head, "kv": kv}

    # -- dense fp32 reference of the same model (decode weights with the GPU's bit-exact decompress) --------
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """Pushes a whole prompt `tokens` [rows, T] through the network in one pass: every block linear runs as the
        fused dequant-GEMM on the tensor cores (rows x T tokens at once), the KV caches are filled for positions
        0..T-1, `pos` is set to T and `ids` to the greedy choice after the last prompt token.  Returns the logits of
        the last position, fp16 [rows, vocab].  Attention over the prompt is torch's scaled_dot_product_attention;
        norms, transforms, RoPE + cache writes, residual adds and the gated-MLP middle are this library's glue
        kernels; decoding continues with `step`."""
        cfg = self.cfg
        R, T = tokens.shape
        if R != self.rows or T > cfg.max_pos:
            raise ValueError("tokens must be [rows, T] with T <= max_pos")
        D = cfg.head_dim
        q_dim = self.heads_l * D
        h = self.embed[tokens.long()].reshape(R * T, cfg.hidden)                     # fp16 residual stream

        def reduce(y):
            if self.tp_world > 1:
                import torch.distributed as dist
                dist.all_reduce(y, group=self.tp_group)
            return y

        xn = torch.empty_like(h)
        for i, b in enumerate(self.blocks):
            ops.rmsnorm(h, b.norm1, xn, cfg.rms_eps)
            qkv = b.qkv(xn)
            ops.rope_cache_prompt(qkv, R, T, self.kcache[i], self.vcache[i], self.heads_l, self.kv_heads_l, D, cfg.rope_theta)
            q = qkv[:, :q_dim].reshape(R, T, self.heads_l, D)                        # rotated in place
            k, v = self.kcache[i][:, :T], self.vcache[i][:, :T]
            att = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                                   is_causal=True, enable_gqa=self.heads_l != self.kv_heads_l)
            att = att.transpose(1, 2).reshape(R * T, q_dim)
            fused = b.o.incoherent and R * T > 8 and self.tp_world == 1       # residual and SwiGLU inside the glue kernels
            if fused:
                h = b.o.finish_t(b.o.product_t(b.o.transform_in(att)), residual=h)
            else:
                h = h + reduce(b.o(att))
            ops.rmsnorm(h, b.norm2, xn, cfg.rms_eps)
            if fused:
                gu = b.gate_up.product_t(b.gate_up.transform_in(xn))                  # before gate-up's output transform
                mlp_t = ops.swiglu_hadamard_f16(gu, torch.empty((R * T, self.ffn_l), dtype=torch.float16, device=self.device),
                                                b.gate_up.signs_out, b.down.signs_in, self.ffn_l, b.down.block_in, b.gate_up.scale)
                h = b.down.finish_t(b.down.product_t(mlp_t), residual=h)
            else:
                gu = b.gate_up(xn)
                mlp = torch.nn.functional.silu(gu[:, : self.ffn_l]).mul_(gu[:, self.ffn_l:])      # fp32 inside, fp16 in and out
                h = h + reduce(b.down(mlp))
        last = h.reshape(R, T, cfg.hidden)[:, -1].contiguous()
        ops.rmsnorm(last, self.norm_f, self.xn, cfg.rms_eps)
        ops.dense_gemv(self.head, self.xn, out=self.logits)
        self.pos.fill_(T - 1)
        self._pos_hi = T
        ops.next_token(self.logits, self.next_ids, self.ids, self.pos, None)        # pos -> T, ids -> greedy choice
        return self.logits

    def reference_logits(self, tokens: torch.Tensor, act_dtype: torch.dtype | None = None) -> torch.Tensor:
        """fp32 torch forward of the same network on `tokens` [rows, T] -> logits [rows, T, vocab].

        act_dtype = torch.float16 gives the yardstick of a stock half-precision evaluation instead: the same fp32 arithmetic,
        but every activation that a half-precision model stores (the normalised layer inputs, q/k/v, the attention output,
        the gated-MLP middle, the residual stream) is rounded to fp16 where it is stored."""
        cfg = self.cfg
        T = tokens.shape[1]
        rnd = (lambda t: t) if act_dtype is None else (lambda t: t.to(act_dtype).float())
        h = self.embed[tokens.long()].float()
        half = cfg.head_dim // 2
        inv = cfg.rope_theta ** (-torch.arange(half, device=self.device, dtype=torch.float32) * 2 / cfg.head_dim)
        ang = torch.arange(T, device=self.device, dtype=torch.float32)[:, None] * inv[None, :]
        cs, sn = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

        def rms(x, w):
            return rnd(x * torch.rsqrt((x * x).mean(-1, keepdim=True) + cfg.rms_eps) * w.float())

        def rope(x):
            a, b = x[..., :half], x[..., half:]
            return rnd(torch.cat((a * cs - b * sn, b * cs + a * sn), dim=-1))

        q_dim, kv_dim = self.heads_l * cfg.head_dim, self.kv_heads_l * cfg.head_dim
        mask = torch.full((T, T), float("-inf"), device=self.device).triu(1)

        def reduce(t):
            if self.tp_world > 1:
                import torch.distributed as dist
                dist.all_reduce(t, group=self.tp_group)
            return t

        for b in self.blocks:
            x = rms(h, b.norm1)
            qkv = rnd(x @ b.qkv.effective_weight().t())
            q = rope(qkv[..., :q_dim].reshape(-1, T, self.heads_l, cfg.head_dim))
            k = rope(qkv[..., q_dim:q_dim + kv_dim].reshape(-1, T, self.kv_heads_l, cfg.head_dim))
            v = qkv[..., q_dim + kv_dim:].reshape(-1, T, self.kv_heads_l, cfg.head_dim)
            rep = self.heads_l // self.kv_heads_l
            k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
            att = torch.einsum("bthd,bshd->bhts", q, k) * cfg.head_dim ** -0.5 + mask
            o = rnd(torch.einsum("bhts,bshd->bthd", att.softmax(-1), v).reshape(-1, T, q_dim))
            h = rnd(h + reduce(o @ b.o.effective_weight().t()))
            x = rms(h, b.norm2)
            gu = rnd(x @ b.gate_up.effective_weight().t())
            h = rnd(h + reduce(rnd(torch.nn.functional.silu(gu[..., : self.ffn_l]) * gu[..., self.ffn_l:]) @ b.down.effective_weight().t()))
        return rms(h, self.norm_f) @ self.head.float().t()


class HostTokenLoop:
    """Greedy decoding with the host in the loop: every step's input ids come from host memory and every step's
    chosen ids go back to it, yet the GPU does not idle while the host turns a token around.

    The host keeps one graph launch queued ahead.  The queued step's first kernel waits (bounded) for the mailbox
    entry that carries its sequence number; the host posts it as soon as it has read the previous step's result from
    the outgoing mailbox, which the step's last kernel writes.  Per step: one 8-byte store by the host that the GPU
    reads over PCIe, and one 8-byte store by the GPU that the host polls."""

    def __init__(self, model: RPTCLlama, timeout_ms: int = 2000):
        import numpy as np
        self.model = model
        self.slots_in, self.slots_out = model.bind_mailbox(timeout_ms)
        self._in, self._out = self.slots_in.numpy(), self.slots_out.numpy()       # views of the pinned buffers
        self._np = np
        self.seq = 0                       # steps completed (== the device's counter once the stream drains)
        self.timeout_s = timeout_ms * 1e-3
        model.capture(pdl=True)

    def _post(self, seq: int, ids) -> None:
        for r in range(self.model.rows):
            self._in[r] = (seq << 32) | int(ids[r])

    def _await(self, seq: int):
        import time
        deadline = None
        out = self._out
        while True:
            vals = [int(v) for v in out]
            if all((v >> 32) == seq for v in vals):
                return [v & 0xFFFFFFFF for v in vals]
            if deadline is None:
                deadline = time.perf_counter() + self.timeout_s + 5.0
            elif time.perf_counter() > deadline:
                raise TimeoutError(f"no result for step {seq}")

    def run(self, first_ids, n_steps: int) -> list[list[int]]:
        """Decodes n_steps tokens per row starting from `first_ids`; returns the chosen ids, one list per step."""
        model, tokens = self.model, []
        if n_steps <= 0:
            return tokens
        model._claim_positions(n_steps)
        self._post(self.seq + 1, first_ids)
        model.graph.replay()
        for i in range(n_steps):
            more = i + 1 < n_steps
            if more:
                model.graph.replay()               # queued behind the running step; waits for its mailbox entry
            got = self._await(self.seq + 1)
            self.seq += 1
            tokens.append(got)
            if more:
                self._post(self.seq + 1, got)
        return tokens
