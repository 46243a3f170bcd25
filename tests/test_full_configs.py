"""Full-size parity of the two sharded benchmark configurations against the CPU oracle (x.float() @ wire.dequant(...).T,
htr/wire.py:105-113), on one GPU:

  LM head   151936 x 4096, K4 (htr/lmhead.py:9-11: rows are independent per 128-row block), batch 1 and 8
  MoE       experts 4096 -> 2 x 1536 -> 4096, K3, gate and up fused under one input sign vector (htr/moe_encode.py:181-196),
            8 experts, 1 and 32 tokens, through the device-routed grouped launches

Tolerances as in tests/test_gpu_parity.py: float32 <= 1e-5 norm-relative; bf16 <= 4e-3 norm-relative and
|err| <= 2^-7 |y| + 1e-2 rms(y) elementwise.  Batches above four rows run on the tensor-core GEMM: biased fp16 operands
(1024 + byte sum, the reference's own scheme, htr_kernels.cu:312-313) accumulated in float32 and unbiased afterwards, which
costs a few bits to cancellation on long rows: float32 <= 2e-4 there (the reference's fp16-activation kernels sit at 2.1e-4).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def check_bf16(y, ref):
    y = y.float().cpu().numpy()
    assert rel(y, ref) <= 4e-3
    rms = float(np.sqrt(np.mean(np.square(ref))))
    assert np.all(np.abs(y - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-2 * rms)


@pytest.fixture(scope="module")
def lm_head():
    from htr_b200 import wire

    return wire.random_packed(151936, 4096, 4, seed=3004)


@pytest.mark.parametrize("M", (1, 8))
def test_lm_head_against_oracle(coracle, lm_head, M):
    from htr_b200 import ops
    from htr_b200.sharded import RowShardedLinear

    dev = torch.device("cuda:0")
    packed = [t.numpy() for t in lm_head]
    args = [t.to(dev) for t in lm_head]
    x = torch.randn(M, 4096, generator=torch.Generator().manual_seed(40 + M))
    ref = coracle.linear(x.numpy(), *packed)
    y = ops.linear(x.to(dev), *args)
    assert rel(y.cpu().numpy(), ref) <= (1e-5 if M <= 4 else 2e-4)
    xb = x.bfloat16()
    refb = coracle.linear(xb.float().numpy(), *packed)
    yb = ops.linear(xb.to(dev), *args)
    check_bf16(yb, refb)
    # the sharded module on one rank (one run of all 1187 row blocks) asks for the integer-exact kernel, whose sums do not depend on
    # the launch decomposition: equal bit for bit to the operator under the same flag, and within the same tolerances of the oracle
    lin = RowShardedLinear(*lm_head, device=dev)
    with ops.exact_sums():
        yx = ops.linear(xb.to(dev), *args)
    assert torch.equal(lin(xb.to(dev)), yx)
    check_bf16(yx, refb)


def _experts(E, h, inter, K, seed):
    from htr_b200 import wire

    out = []
    for e in range(E):
        out.append(dict(gate_up=wire.random_packed(2 * inter, h, K, seed=seed + 10 * e), down=wire.random_packed(h, inter, K, seed=seed + 10 * e + 1)))
    return out


def _moe_oracle(coracle, experts, x, ids, w):
    """Per expert, the tokens routed to it in one oracle call each for gate_up and down; float64 combine.  Activations between
    the two linears are rounded to x's dtype, as the layer does."""
    T, h = x.shape
    out = np.zeros((T, h), dtype=np.float64)
    for e, ex in enumerate(experts):
        hit = (ids == e).nonzero(as_tuple=False)
        if hit.numel() == 0:
            continue
        tok = hit[:, 0]
        gu = torch.from_numpy(coracle.linear(x[tok].float().numpy(), *[t.numpy() for t in ex["gate_up"]])).to(x.dtype)
        inter = gu.shape[1] // 2
        act = (torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()).to(x.dtype)
        d = torch.from_numpy(coracle.linear(act.float().numpy(), *[t.numpy() for t in ex["down"]])).to(x.dtype)
        for i in range(hit.shape[0]):
            out[int(tok[i])] += float(w[hit[i, 0], hit[i, 1]]) * d[i].double().numpy()
    return out


@pytest.mark.parametrize("T", (1, 32))
def test_moe_experts_against_oracle(coracle, T):
    from htr_b200.sharded import ExpertParallelMoE

    dev = torch.device("cuda:0")
    E, h, inter, K, k = 8, 4096, 1536, 3, 4
    experts = _experts(E, h, inter, K, seed=7000)
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, h, generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    w = torch.rand(T, k, generator=g)
    w = w / w.sum(-1, keepdim=True)
    moe = ExpertParallelMoE(experts, device=dev)
    want = _moe_oracle(coracle, experts, x, ids, w)
    y = moe(x.to(dev), ids, w, grouped=True).float().cpu().numpy()
    assert rel(y, want) <= 1e-5
    y_loop = moe(x.to(dev), ids, w, grouped=False).float().cpu().numpy()
    assert rel(y_loop, want) <= 2e-4        # host routing batches an expert's tokens: above four rows the tensor-core GEMM serves them
    xb = x.bfloat16()
    wantb = _moe_oracle(coracle, experts, xb, ids, w)
    yb = moe(xb.to(dev), ids, w, grouped=True).float().cpu().numpy()
    assert rel(yb, wantb) <= 1e-2          # two bf16 roundings in a row (hidden activation, expert output) before the float32 combine
