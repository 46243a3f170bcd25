"""The packed decoder harness against the same network evaluated with dense weights (decoded by the dequant kernel) in
float32 torch ops: same prompt, same greedy continuation, logits close."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_small_decoder_matches_dense_evaluation():
    from htr_b200 import wire
    from htr_b200.decoder import DecoderConfig, PackedDecoder, _rms_norm

    dev = torch.device("cuda:0")
    cfg = DecoderConfig(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=128, intermediate=512, vocab=1024, K=4, K_head=4, max_len=64)
    model = PackedDecoder(cfg, dev, seed=3)
    # the fused glue kernels reproduce the plain torch ops: same logits for a prompt pass and a single-token step
    plain = PackedDecoder(cfg, dev, seed=3, fused=False)
    ids9 = torch.randint(0, cfg.vocab, (9,), generator=torch.Generator().manual_seed(5)).to(dev)
    lf, lp = model.forward(ids9, torch.arange(9, device=dev)), plain.forward(ids9, torch.arange(9, device=dev))
    assert float((lf.float() - lp.float()).norm() / lp.float().norm()) <= 2e-2
    one, at = ids9[:1], torch.full((1,), 9, device=dev, dtype=torch.long)
    lf1, lp1 = model.forward(one, at), plain.forward(one, at)
    assert float((lf1.float() - lp1.float()).norm() / lp1.float().norm()) <= 2e-2
    assert torch.allclose(model.k_cache.float(), plain.k_cache.float(), atol=2e-2) and torch.allclose(model.v_cache.float(), plain.v_cache.float(), atol=2e-2)
    model = PackedDecoder(cfg, dev, seed=3)
    prompt = torch.randint(0, cfg.vocab, (9,), generator=torch.Generator().manual_seed(1))
    toks, t_prompt, t_decode = model.generate(prompt, 12, use_graph=True)
    toks_eager, _, _ = PackedDecoder(cfg, dev, seed=3).generate(prompt, 12, use_graph=False)
    assert torch.equal(toks, toks_eager)                       # graph replay == eager stepping

    # dense float32 evaluation of the whole sequence (prompt + generated tokens) in one causal pass
    seq = torch.cat([prompt.to(dev), toks[:-1]])
    T = seq.numel()
    dense = lambda w: wire.dequant(*w, dtype=torch.float32)
    x = model.embed[seq].float()
    pos = torch.arange(T, device=dev)
    causal = (pos[None, :] <= pos[:, None])[None, None]
    rep = cfg.q_heads // cfg.kv_heads
    for L in model.layers:
        h = _rms_norm(x, L["ln1"].float(), cfg.eps)
        qkv = h @ dense(L["qkv"]).T
        q, k, v = qkv.split((cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim), dim=-1)
        q = model._rope(q.view(T, cfg.q_heads, cfg.head_dim), pos).permute(1, 0, 2)[None]
        k = model._rope(k.view(T, cfg.kv_heads, cfg.head_dim), pos).permute(1, 0, 2).repeat_interleave(rep, 0)[None]
        v = v.view(T, cfg.kv_heads, cfg.head_dim).permute(1, 0, 2).repeat_interleave(rep, 0)[None]
        att = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=causal)[0].permute(1, 0, 2).reshape(T, -1)
        x = x + att @ dense(L["o"]).T
        h = _rms_norm(x, L["ln2"].float(), cfg.eps)
        gu = h @ dense(L["gate_up"]).T
        x = x + (torch.nn.functional.silu(gu[:, :cfg.intermediate]) * gu[:, cfg.intermediate:]) @ dense(L["down"]).T
    logits = _rms_norm(x, model.ln_f.float(), cfg.eps) @ dense(model.head).T
    # positions len(prompt)-1 .. T-1 predicted the generated tokens
    pred = logits[prompt.numel() - 1:].argmax(-1)
    agree = (pred == toks).float().mean().item()
    assert agree >= 0.75, agree                                 # bf16 chain vs float32: near-ties may flip, most tokens agree
    assert model.packed_bytes_per_token() > 0 and t_decode > 0


@pytest.mark.parametrize("K", (2, 3, 4, 5))
@pytest.mark.parametrize("rows", (1, 3, 8))
def test_folded_gemv_forms_equal_the_separate_kernels(K, rows, monkeypatch):
    """htr_linear_fused against glue kernel + htr_linear: SwiGLU prologue and residual epilogue bit for bit, RMSNorm prologue
    up to the summation order of the row's mean square (<= 1 bf16 ulp on a few inputs)."""
    from htr_b200 import _lib, ops, wire

    monkeypatch.setattr(ops, "GEMV_ROUTE_MAX", 8)
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream(dev).cuda_stream
    n, m = 512, 384
    g = torch.Generator().manual_seed(10 * K + rows)
    w = wire.random_packed(m, n, K, seed=K + rows, device=dev)
    x = torch.randn(rows, n, generator=g).bfloat16().to(dev)
    gamma = (1.0 + 0.1 * torch.randn(n, generator=g)).bfloat16().to(dev)
    # RMSNorm folded into the activation staging
    h = torch.empty_like(x)
    resid = x.clone()
    _lib.check(_lib.lib.htr_dec_add_rmsnorm(resid.data_ptr(), None, gamma.data_ptr(), h.data_ptr(), rows, n, 1e-6, st), "htr_dec_add_rmsnorm")
    want = ops.linear(h, *w)
    got = ops.linear_fused(x, *w, prologue=ops.PROLOGUE_RMSNORM, norm_weight=gamma, eps=1e-6)
    assert float((got.float() - want.float()).norm() / want.float().norm()) <= 2e-3
    assert float((got != want).float().mean()) <= 0.05
    # SwiGLU folded into the activation staging: x = [gate | up]
    w2 = wire.random_packed(m, n, K, seed=50 + K + rows, device=dev)
    gu = torch.randn(rows, 2 * n, generator=g).bfloat16().to(dev)
    act = torch.empty(rows, n, dtype=torch.bfloat16, device=dev)
    _lib.check(_lib.lib.htr_dec_swiglu(gu.data_ptr(), act.data_ptr(), rows, n, st), "htr_dec_swiglu")
    assert torch.equal(ops.linear_fused(gu, *w2, prologue=ops.PROLOGUE_SWIGLU), ops.linear(act, *w2))
    # residual epilogue: out += result, in place
    stream = torch.randn(rows, m, generator=g).bfloat16().to(dev)
    want = stream + ops.linear(x, *w)
    out = stream.clone()
    assert ops.linear_fused(x, *w, out=out, residual=True) is out and torch.equal(out, want)
    # both at once, as the down projection uses them
    want = stream + ops.linear(act, *w2)
    out = stream.clone()
    ops.linear_fused(gu, *w2, out=out, prologue=ops.PROLOGUE_SWIGLU, residual=True)
    assert torch.equal(out, want)
    with pytest.raises(_lib.HTRError):
        ops.linear_fused(x.float(), *w)
    with pytest.raises(_lib.HTRError):
        ops.linear_fused(x, *w, residual=True)
    with pytest.raises(_lib.HTRError):
        ops.linear_fused(x, *w, prologue=ops.PROLOGUE_RMSNORM)          # no norm weight


def test_single_token_rope_attention_equals_the_two_kernels():
    from htr_b200 import _lib

    dev = torch.device("cuda:0")
    L = _lib.lib
    st = torch.cuda.current_stream(dev).cuda_stream
    hq, hkv, D, max_len = 8, 2, 128, 300
    g = torch.Generator().manual_seed(3)
    inv = 1.0 / (1.0e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(max_len).float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(dev), ang.sin().to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for p in (0, 1, 7, 130, 299):                                           # 299 = the last row of the caches
        kc = torch.randn(max_len, hkv, D, generator=g).bfloat16().to(dev)
        vc = torch.randn(max_len, hkv, D, generator=g).bfloat16().to(dev)
        qkv = torch.randn(1, (hq + 2 * hkv) * D, generator=g).bfloat16().to(dev)
        pos = torch.full((1,), p, dtype=torch.long, device=dev)
        k1, v1, k2, v2 = kc.clone(), vc.clone(), kc.clone(), vc.clone()
        q = torch.empty(1, hq, D, dtype=torch.bfloat16, device=dev)
        want, got = torch.empty_like(q), torch.empty_like(q)
        _lib.check(L.htr_dec_rope_cache(qkv.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), q.data_ptr(), k1.data_ptr(), v1.data_ptr(),
                                        1, hq, hkv, D, max_len, status.data_ptr(), st), "htr_dec_rope_cache")
        _lib.check(L.htr_dec_attention(q.data_ptr(), k1.data_ptr(), v1.data_ptr(), pos.data_ptr(), want.data_ptr(), 1, hq, hkv, D, max_len,
                                       status.data_ptr(), st), "htr_dec_attention")
        _lib.check(L.htr_dec_rope_attention(qkv.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), k2.data_ptr(), v2.data_ptr(), got.data_ptr(),
                                            hq, hkv, D, max_len, status.data_ptr(), st), "htr_dec_rope_attention")
        assert torch.equal(k1, k2) and torch.equal(v1, v2)                 # the same cache rows
        assert float((got.float() - want.float()).abs().max()) <= 2e-2 * float(want.float().abs().max())
    assert int(status.item()) == 0                                          # every position was inside the caches
