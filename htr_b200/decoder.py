"""Minimal dense decoder whose linears are HTR-W1 packed: the caller that turns packed-GEMV GB/s into decode tokens/s.

Stands in for the model code that surrounds `HTRLinearMethod.apply` in a serving stack (htr/vllm_plugin.py:130-138) for
the reference's headline case: a 9B-class dense decoder (36 layers, hidden 4096, 32 query / 8 KV heads of 128, SwiGLU
12288, vocabulary 151936), every trunk linear and the LM head packed, norms and embeddings bf16, one sequence, greedy
decoding (docs/case-studies/dense-9b.md of the reference).  Weights are random (no checkpoint is available); fused
projections (q|k|v, gate|up) are single packed linears, as the format prescribes (docs/FORMAT.md:31-32).

Every packed linear goes through `htr_b200.ops.linear`.  The glue between them (residual add + RMSNorm, rotary embedding
+ KV-cache write, single-query grouped attention, SwiGLU) runs as four small fused kernels of the library
(`htr_dec_*`, launched with programmatic stream serialisation so the following packed GEMV prefetches its weights while
they run); `fused=False` evaluates the same glue with plain torch ops, which is how the kernels are checked.  Steps of at
most 8 rows (decoding) fold the norms, the SwiGLU and the residual adds into the packed GEMVs themselves
(`ops.linear_fused`) and, for a single token, the rotary embedding and cache write into the attention kernel: five launches
per layer.  A decode step reads its position from a device tensor, so one CUDA graph captured once serves every step.
"""
import dataclasses
import math

import torch

from . import _lib, ops, wire


@dataclasses.dataclass
class DecoderConfig:
    layers: int = 36
    hidden: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 12288
    vocab: int = 151936
    K: int = 4                 # bits per weight of the trunk
    K_head: int = 4            # bits per weight of the LM head
    max_len: int = 512
    rope_theta: float = 1.0e6
    eps: float = 1.0e-6


def _rms_norm(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class PackedDecoder:
    def __init__(self, cfg, device, seed=0, dtype=torch.bfloat16, fused=True, weights=None):
        """Random packed weights from `seed`, or `weights` = dict(layers=[{qkv, o, gate_up, down, ln1, ln2}], head, ln_f, embed)
        already on `device` (see from_checkpoint)."""
        self.cfg, self.device, self.dtype, self.fused = cfg, device, dtype, fused
        self.fold = True                                       # decode-sized steps: fold norms / SwiGLU / residual adds into the GEMVs
        assert cfg.max_len <= 1024, "the attention glue kernel holds at most 1024 positions"
        c = cfg
        if weights is None:
            weights = self.random_weights(cfg, device, seed, dtype)
        self.layers, self.head, self.ln_f, self.embed = weights["layers"], weights["head"], weights["ln_f"], weights["embed"]
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2).float() / c.head_dim))
        ang = torch.arange(c.max_len).float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos().to(device), ang.sin().to(device)
        self.k_cache = torch.zeros(c.layers, c.max_len, c.kv_heads, c.head_dim, dtype=dtype, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.arange = torch.arange(c.max_len, device=device)
        # set by the glue kernels when a position lies outside the caches (htr_dec_rope_cache / _attention / _rope_attention)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    @staticmethod
    def random_weights(cfg, device, seed=0, dtype=torch.bfloat16):
        g = torch.Generator().manual_seed(seed)
        c = cfg
        qkv_out = (c.q_heads + 2 * c.kv_heads) * c.head_dim

        def packed(m, n, K, s):
            return wire.random_packed(m, n, K, seed=seed * 100003 + s, device=device)

        layers = []
        for i in range(c.layers):
            layers.append(dict(
                qkv=packed(qkv_out, c.hidden, c.K, 10 * i + 1), o=packed(c.hidden, c.q_heads * c.head_dim, c.K, 10 * i + 2),
                gate_up=packed(2 * c.intermediate, c.hidden, c.K, 10 * i + 3), down=packed(c.hidden, c.intermediate, c.K, 10 * i + 4),
                ln1=torch.ones(c.hidden, dtype=dtype, device=device), ln2=torch.ones(c.hidden, dtype=dtype, device=device)))
        return dict(layers=layers, head=packed(c.vocab, c.hidden, c.K_head, 7), ln_f=torch.ones(c.hidden, dtype=dtype, device=device),
                    embed=(torch.randn(c.vocab, c.hidden, generator=g) * 0.02).to(dtype).to(device))

    # ---- checkpoints in the reference converter's layout (htr_b200/checkpoint.py) ----------------------------------
    def export_checkpoint(self, out_dir, shards=2):
        """Writes this model as a packed checkpoint: fused projections are stored per member (q/k/v, gate/up), as the
        reference's converter stores them (htr/quantize.py:252-289)."""
        from . import checkpoint

        c = self.cfg
        packed, plain = {}, {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.ln_f}

        def members(t, sizes, names, prefix):
            qw, sc, su, sv = t
            at = 0
            for name, rows in zip(names, sizes):
                packed[f"{prefix}.{name}"] = (qw[at // 16:(at + rows) // 16], sc[at:at + rows], su, sv[at // 8:(at + rows) // 8])
                at += rows

        for i, L in enumerate(self.layers):
            pre = f"model.layers.{i}"
            members(L["qkv"], [c.q_heads * c.head_dim, c.kv_heads * c.head_dim, c.kv_heads * c.head_dim], ["q_proj", "k_proj", "v_proj"],
                    f"{pre}.self_attn")
            packed[f"{pre}.self_attn.o_proj"] = L["o"]
            members(L["gate_up"], [c.intermediate, c.intermediate], ["gate_proj", "up_proj"], f"{pre}.mlp")
            packed[f"{pre}.mlp.down_proj"] = L["down"]
            plain[f"{pre}.input_layernorm.weight"] = L["ln1"]
            plain[f"{pre}.post_attention_layernorm.weight"] = L["ln2"]
        packed["lm_head"] = self.head
        config = dict(architectures=["PackedDecoder"], num_hidden_layers=c.layers, hidden_size=c.hidden, num_attention_heads=c.q_heads,
                      num_key_value_heads=c.kv_heads, head_dim=c.head_dim, intermediate_size=c.intermediate, vocab_size=c.vocab,
                      rope_theta=c.rope_theta, rms_norm_eps=c.eps, max_position_embeddings=c.max_len, torch_dtype="bfloat16")
        return checkpoint.write_checkpoint(out_dir, packed, plain, config, shards=shards)

    @classmethod
    def from_checkpoint(cls, ckpt_dir, device, fused=True, dtype=torch.bfloat16):
        """Builds the model from a packed checkpoint through the serving plugin: `HTRConfig.from_config` picks the method per
        module, `HTRLinearMethod.create_weights` allocates the fused parameters, and every checkpoint tensor reaches them
        through their `weight_loader` (htr/vllm_plugin.py:40-125 of the reference)."""
        from vllm.model_executor.layers.linear import LinearBase

        from . import checkpoint, vllm_plugin

        hf = checkpoint.read_config(ckpt_dir)
        qc = vllm_plugin.HTRConfig.from_config(hf["quantization_config"])
        qc.packed_modules_mapping = {"qkv_proj": ["q_proj", "k_proj", "v_proj"], "gate_up_proj": ["gate_proj", "up_proj"]}
        c = DecoderConfig(layers=hf["num_hidden_layers"], hidden=hf["hidden_size"], q_heads=hf["num_attention_heads"],
                          kv_heads=hf["num_key_value_heads"], head_dim=hf["head_dim"], intermediate=hf["intermediate_size"],
                          vocab=hf["vocab_size"], max_len=hf.get("max_position_embeddings", 512), rope_theta=hf["rope_theta"],
                          eps=hf["rms_norm_eps"])
        params, holders = {}, {}

        def linear(prefix, n, sizes, lm_head=False):
            holder = LinearBase.__new__(LinearBase)            # only its type matters to get_quant_method
            torch.nn.Module.__init__(holder)
            method = vllm_plugin.HTRLinearMethod(qc.modules["lm_head"]) if lm_head else qc.get_quant_method(holder, prefix)
            assert isinstance(method, vllm_plugin.HTRLinearMethod), f"{prefix} is not packed in this checkpoint"
            method.create_weights(holder, n, sizes, n, sum(sizes), dtype)
            for leaf in ("htr_qweight", "htr_scales", "htr_su", "htr_sv"):
                params[f"{prefix}.{leaf}"] = getattr(holder, leaf)
            holders[prefix] = holder
            return holder

        def plain(name, shape):
            params[name] = torch.nn.Parameter(torch.empty(shape, dtype=dtype), requires_grad=False)
            return params[name]

        plain("model.embed_tokens.weight", (c.vocab, c.hidden))
        plain("model.norm.weight", (c.hidden,))
        for i in range(c.layers):
            pre = f"model.layers.{i}"
            linear(f"{pre}.self_attn.qkv_proj", c.hidden, [c.q_heads * c.head_dim, c.kv_heads * c.head_dim, c.kv_heads * c.head_dim])
            linear(f"{pre}.self_attn.o_proj", c.q_heads * c.head_dim, [c.hidden])
            linear(f"{pre}.mlp.gate_up_proj", c.hidden, [c.intermediate, c.intermediate])
            linear(f"{pre}.mlp.down_proj", c.intermediate, [c.hidden])
            plain(f"{pre}.input_layernorm.weight", (c.hidden,))
            plain(f"{pre}.post_attention_layernorm.weight", (c.hidden,))
        linear("lm_head", c.hidden, [c.vocab], lm_head=True)
        got = checkpoint.load_checkpoint(ckpt_dir, params)
        missing = sorted(set(params) - got)
        assert not missing, f"checkpoint lacks {missing[:4]}"

        def tensors(prefix):
            h = holders[prefix]
            return tuple(t.data.to(device) for t in (h.htr_qweight, h.htr_scales, h.htr_su, h.htr_sv))

        K_trunk = holders["model.layers.0.self_attn.qkv_proj"].htr_K if c.layers else 4
        c.K, c.K_head = K_trunk, holders["lm_head"].htr_K
        layers = []
        for i in range(c.layers):
            pre = f"model.layers.{i}"
            layers.append(dict(qkv=tensors(f"{pre}.self_attn.qkv_proj"), o=tensors(f"{pre}.self_attn.o_proj"),
                               gate_up=tensors(f"{pre}.mlp.gate_up_proj"), down=tensors(f"{pre}.mlp.down_proj"),
                               ln1=params[f"{pre}.input_layernorm.weight"].data.to(device),
                               ln2=params[f"{pre}.post_attention_layernorm.weight"].data.to(device)))
        weights = dict(layers=layers, head=tensors("lm_head"), ln_f=params["model.norm.weight"].data.to(device),
                       embed=params["model.embed_tokens.weight"].data.to(device))
        return cls(c, device, dtype=dtype, fused=fused, weights=weights)

    def packed_bytes_per_token(self):
        """Packed payload read by one decode step (every trunk linear once + the LM head)."""
        c = self.cfg
        qkv_out = (c.q_heads + 2 * c.kv_heads) * c.head_dim
        per_layer = (wire.payload_bytes(qkv_out, c.hidden, c.K) + wire.payload_bytes(c.hidden, c.q_heads * c.head_dim, c.K) +
                     wire.payload_bytes(2 * c.intermediate, c.hidden, c.K) + wire.payload_bytes(c.hidden, c.intermediate, c.K))
        return c.layers * per_layer + wire.payload_bytes(c.vocab, c.hidden, c.K_head)

    def _rope(self, t, pos):
        cos, sin = self.cos.index_select(0, pos)[:, None, :], self.sin.index_select(0, pos)[:, None, :]
        t1, t2 = t[..., ::2].float(), t[..., 1::2].float()
        out = torch.stack((t1 * cos - t2 * sin, t1 * sin + t2 * cos), dim=-1)
        return out.flatten(-2).to(t.dtype)

    def forward_fused(self, ids, pos):
        """The same step with the library's glue kernels (bf16 only)."""
        c, L_ = self.cfg, _lib.lib
        T = ids.shape[0]
        if T <= ops.GEMV_MAX_M and self.fold:
            return self.forward_folded(ids, pos)
        dev = self.device
        st = torch.cuda.current_stream(dev).cuda_stream
        x = self.embed.index_select(0, ids)                     # residual stream, updated in place
        h = torch.empty_like(x)
        q = torch.empty(T, c.q_heads, c.head_dim, dtype=self.dtype, device=dev)
        att = torch.empty_like(q)
        act = torch.empty(T, c.intermediate, dtype=self.dtype, device=dev)
        delta = None
        for li, L in enumerate(self.layers):
            _lib.check(L_.htr_dec_add_rmsnorm(x.data_ptr(), None if delta is None else delta.data_ptr(), L["ln1"].data_ptr(), h.data_ptr(),
                                              T, c.hidden, c.eps, st), "htr_dec_add_rmsnorm")
            qkv = ops.linear(h, *L["qkv"])
            _lib.check(L_.htr_dec_rope_cache(qkv.data_ptr(), pos.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), q.data_ptr(),
                                             self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr(), T, c.q_heads, c.kv_heads, c.head_dim,
                                             c.max_len, self.status.data_ptr(), st), "htr_dec_rope_cache")
            _lib.check(L_.htr_dec_attention(q.data_ptr(), self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr(), pos.data_ptr(),
                                            att.data_ptr(), T, c.q_heads, c.kv_heads, c.head_dim, c.max_len, self.status.data_ptr(), st),
                       "htr_dec_attention")
            o = ops.linear(att.view(T, c.q_heads * c.head_dim), *L["o"])
            _lib.check(L_.htr_dec_add_rmsnorm(x.data_ptr(), o.data_ptr(), L["ln2"].data_ptr(), h.data_ptr(), T, c.hidden, c.eps, st),
                       "htr_dec_add_rmsnorm")
            gu = ops.linear(h, *L["gate_up"])
            _lib.check(L_.htr_dec_swiglu(gu.data_ptr(), act.data_ptr(), T, c.intermediate, st), "htr_dec_swiglu")
            delta = ops.linear(act, *L["down"])
        _lib.check(L_.htr_dec_add_rmsnorm(x.data_ptr(), delta.data_ptr(), self.ln_f.data_ptr(), h.data_ptr(), T, c.hidden, c.eps, st),
                   "htr_dec_add_rmsnorm")
        return ops.linear(h, *self.head)

    def forward_folded(self, ids, pos):
        """Decode-sized step (at most 8 rows) with the norms, the SwiGLU and the residual adds folded into the packed GEMVs
        (`ops.linear_fused`): six launches per layer instead of nine, five for a single token."""
        c, L_ = self.cfg, _lib.lib
        T = ids.shape[0]
        dev = self.device
        st = torch.cuda.current_stream(dev).cuda_stream
        x = self.embed.index_select(0, ids)                     # residual stream, updated in place by the o and down projections
        q = torch.empty(T, c.q_heads, c.head_dim, dtype=self.dtype, device=dev)
        att = torch.empty_like(q)
        for li, L in enumerate(self.layers):
            qkv = ops.linear_fused(x, *L["qkv"], prologue=ops.PROLOGUE_RMSNORM, norm_weight=L["ln1"], eps=c.eps)
            if T == 1:                                          # one token: rotary embedding, cache write and attention in one launch
                _lib.check(L_.htr_dec_rope_attention(qkv.data_ptr(), pos.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(),
                                                     self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr(), att.data_ptr(),
                                                     c.q_heads, c.kv_heads, c.head_dim, c.max_len, self.status.data_ptr(), st),
                           "htr_dec_rope_attention")
            else:
                _lib.check(L_.htr_dec_rope_cache(qkv.data_ptr(), pos.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), q.data_ptr(),
                                                 self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr(), T, c.q_heads, c.kv_heads, c.head_dim,
                                                 c.max_len, self.status.data_ptr(), st), "htr_dec_rope_cache")
                _lib.check(L_.htr_dec_attention(q.data_ptr(), self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr(), pos.data_ptr(),
                                                att.data_ptr(), T, c.q_heads, c.kv_heads, c.head_dim, c.max_len, self.status.data_ptr(), st),
                       "htr_dec_attention")
            ops.linear_fused(att.view(T, c.q_heads * c.head_dim), *L["o"], out=x, residual=True)
            gu = ops.linear_fused(x, *L["gate_up"], prologue=ops.PROLOGUE_RMSNORM, norm_weight=L["ln2"], eps=c.eps)
            ops.linear_fused(gu, *L["down"], out=x, prologue=ops.PROLOGUE_SWIGLU, residual=True)
        return ops.linear_fused(x, *self.head, prologue=ops.PROLOGUE_RMSNORM, norm_weight=self.ln_f, eps=c.eps)

    def forward(self, ids, pos):
        """ids [T] token ids, pos [T] their positions (device tensors).  Returns logits [T, vocab] and updates the cache."""
        c = self.cfg
        if self.fused and self.dtype == torch.bfloat16 and c.head_dim == 128:
            return self.forward_fused(ids, pos)
        T = ids.shape[0]
        x = self.embed.index_select(0, ids)
        # a query at position p sees cache slots <= p
        mask = (self.arange[None, :] <= pos[:, None])[None, None]                     # [1, 1, T, max_len]
        rep = c.q_heads // c.kv_heads
        for li, L in enumerate(self.layers):
            h = _rms_norm(x, L["ln1"], c.eps)
            qkv = ops.linear(h, *L["qkv"])
            q, k, v = qkv.split((c.q_heads * c.head_dim, c.kv_heads * c.head_dim, c.kv_heads * c.head_dim), dim=-1)
            q = self._rope(q.view(T, c.q_heads, c.head_dim), pos)
            k = self._rope(k.view(T, c.kv_heads, c.head_dim), pos)
            self.k_cache[li].index_copy_(0, pos, k)
            self.v_cache[li].index_copy_(0, pos, v.view(T, c.kv_heads, c.head_dim))
            kk = self.k_cache[li].permute(1, 0, 2).repeat_interleave(rep, dim=0)[None]   # [1, q_heads, max_len, d]
            vv = self.v_cache[li].permute(1, 0, 2).repeat_interleave(rep, dim=0)[None]
            att = torch.nn.functional.scaled_dot_product_attention(q.permute(1, 0, 2)[None], kk, vv, attn_mask=mask)
            x = x + ops.linear(att[0].permute(1, 0, 2).reshape(T, c.q_heads * c.head_dim), *L["o"])
            h = _rms_norm(x, L["ln2"], c.eps)
            gu = ops.linear(h, *L["gate_up"])
            act = torch.nn.functional.silu(gu[:, :c.intermediate]) * gu[:, c.intermediate:]
            x = x + ops.linear(act, *L["down"])
        return ops.linear(_rms_norm(x, self.ln_f, c.eps), *self.head)

    @torch.no_grad()
    def generate(self, prompt_ids, new_tokens, use_graph=True):
        """Greedy decoding: one forward over the prompt (batched rows), then `new_tokens` single-token steps.
        Returns (token ids [new_tokens], seconds for the prompt, seconds for the decode steps) measured with CUDA events."""
        dev = self.device
        P = prompt_ids.numel()
        assert P + new_tokens <= self.cfg.max_len
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        cur = torch.zeros(1, dtype=torch.long, device=dev)
        pos = torch.zeros(1, dtype=torch.long, device=dev)
        out = torch.zeros(new_tokens, dtype=torch.long, device=dev)

        def step():
            logits = self.forward(cur, pos)
            cur.copy_(logits.argmax(-1))
            pos.add_(1)

        graph = None
        if use_graph:                                    # warm up and capture before the timed region (cache content is rewritten below)
            cur.zero_(); pos.fill_(P)
            step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            torch.cuda.synchronize()
        ev[0].record()
        logits = self.forward(prompt_ids.to(dev), torch.arange(P, device=dev))
        cur.copy_(logits[-1:].argmax(-1))
        pos.fill_(P)
        ev[1].record()
        for t in range(new_tokens):
            out[t] = cur[0]
            if graph is not None:
                graph.replay()
            else:
                step()
        ev[2].record()
        torch.cuda.synchronize()
        if int(self.status.item()):
            raise _lib.HTRError(f"a decode step used a position outside the {self.cfg.max_len}-row caches (status {int(self.status.item())})")
        return out, ev[0].elapsed_time(ev[1]) * 1e-3, ev[1].elapsed_time(ev[2]) * 1e-3
