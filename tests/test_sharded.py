"""Row-sharded linears and expert-parallel MoE.  Host-side logic runs as two gloo ranks on CPU with the CPU oracle injected
as the linear; the CUDA cases check the single-rank path against the oracle and, where two GPUs are present, NCCL ranks
against the single-GPU result (bit-identical, as a row block is computed by the same code whichever rank owns it)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_linear():
    from oracle import oracle as O

    co = O.COracle()

    def fn(x, qw, sc, su, sv, bias=None):
        y = co.linear(x.float().numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy(), None if bias is None else bias.float().numpy(), threads=2)
        return torch.from_numpy(y).to(x.dtype)

    return fn


def _moe_inputs(E=4, h=128, inter=128, T=5, k=2, K=3, seed=0):
    from htr_b200 import wire

    experts = []
    for e in range(E):
        gu = wire.random_packed(2 * inter, h, K, seed=seed + 10 * e)
        dn = wire.random_packed(h, inter, K, seed=seed + 10 * e + 1)
        experts.append(dict(gate_up=gu, down=dn))
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, h, generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    w = torch.rand(T, k, generator=g)
    w = w / w.sum(-1, keepdim=True)
    return experts, x, ids, w


def _moe_reference(experts, x, ids, w, fn):
    out = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32)
    for t in range(x.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            gu = fn(x[t:t + 1], *experts[e]["gate_up"])
            inter = gu.shape[1] // 2
            act = (torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()).to(x.dtype)
            out[t] += float(w[t, j]) * fn(act, *experts[e]["down"])[0].float()
    return out


def test_partitions():
    from htr_b200.sharded import expert_partition, row_block_partition

    per, runs = row_block_partition(151936, 8)
    assert per == 149 and runs[0] == (0, 149) and runs[7] == (1043, 144) and sum(r[1] for r in runs) == 1187
    assert row_block_partition(4096, 1) == (32, [(0, 32)])
    per, runs = row_block_partition(384, 4)
    assert per == 1 and runs == [(0, 1), (1, 1), (2, 1), (3, 0)]
    assert expert_partition(64, 8) == [(8 * r, 8) for r in range(8)]
    assert expert_partition(6, 4) == [(0, 2), (2, 2), (4, 2), (6, 0)]
    with pytest.raises(ValueError):
        row_block_partition(100, 2)


def _gloo_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from htr_b200 import wire
        from htr_b200.sharded import ExpertParallelMoE, RowShardedLinear

        fn = _oracle_linear()
        qw, sc, su, sv = wire.random_packed(384, 256, 4, seed=5)           # 3 row blocks over 2 ranks: 2 + (1 real, 1 padding)
        bias = torch.randn(384, generator=torch.Generator().manual_seed(1))
        x = torch.randn(2, 3, 256, generator=torch.Generator().manual_seed(2))
        lin = RowShardedLinear(qw, sc, su, sv, bias=bias, linear_fn=fn)
        assert lin.qweight.shape[0] == 16 and lin.scales.shape[0] == 256
        y = lin(x)
        experts, xm, ids, w = _moe_inputs()
        moe = ExpertParallelMoE(experts, linear_fn=fn)
        assert sorted(moe.local) == [2 * rank, 2 * rank + 1]
        ym = moe(xm, ids, w)
        q.put((rank, y.numpy(), ym.numpy()))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_the_unsharded_result():
    from htr_b200 import wire

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(2):
        rank, y, ym = q.get(timeout=240)
        got[rank] = (y, ym)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    fn = _oracle_linear()
    qw, sc, su, sv = wire.random_packed(384, 256, 4, seed=5)
    bias = torch.randn(384, generator=torch.Generator().manual_seed(1))
    x = torch.randn(2, 3, 256, generator=torch.Generator().manual_seed(2))
    want = fn(x.reshape(6, 256), qw, sc, su, sv, bias).reshape(2, 3, 384).numpy()
    experts, xm, ids, w = _moe_inputs()
    want_moe = _moe_reference(experts, xm, ids, w, fn).numpy()
    for rank in (0, 1):
        y, ym = got[rank]
        assert y.shape == (2, 3, 384)
        assert np.array_equal(y, want)                                       # same code per row block: identical
        assert np.allclose(ym, want_moe, rtol=1e-5, atol=1e-6)
    assert np.array_equal(got[0][1], got[1][1])                              # rank-ordered combine: every rank holds the same bits


@pytest.mark.gpu
def test_single_rank_paths_on_gpu(coracle):
    from htr_b200 import ops, wire
    from htr_b200.sharded import ExpertParallelMoE, RowShardedLinear

    dev = torch.device("cuda:0")
    qw, sc, su, sv = wire.random_packed(1024, 512, 4, seed=3, device=dev)
    x = torch.randn(4, 512, device=dev).bfloat16()
    lin = RowShardedLinear(qw, sc, su, sv)
    assert torch.equal(lin(x), ops.linear(x, qw, sc, su, sv))
    experts, xm, ids, w = _moe_inputs(E=8, h=256, inter=128, T=6, k=2, K=3, seed=4)
    moe = ExpertParallelMoE(experts, device=dev)
    want = _moe_reference(experts, xm, ids, w, _oracle_linear())
    y_loop = moe(xm.to(dev), ids, w, grouped=False).float().cpu()            # host-routed, one call per expert
    y_grp = moe(xm.to(dev), ids, w, grouped=True).float().cpu()              # two grouped launches, routing on the device
    assert float((y_loop - want).norm() / want.norm()) <= 1e-5
    assert float((y_grp - want).norm() / want.norm()) <= 1e-5
    # bf16 tokens through the grouped path, several tokens hitting the same expert
    xb = xm.bfloat16()
    yb = moe(xb.to(dev), ids, w, grouped=True).float().cpu()
    wantb = _moe_reference(experts, xb, ids, w, _oracle_linear())
    assert float((yb - wantb).norm() / wantb.norm()) <= 1e-2


def _nccl_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from htr_b200 import ops, wire
        from htr_b200.sharded import RowShardedLinear

        qw, sc, su, sv = wire.random_packed(128 * 11, 1024, 4, seed=8)      # 11 row blocks over 2 ranks: 6 + (5 real, 1 padding)
        x = torch.randn(3, 1024, generator=torch.Generator().manual_seed(9)).bfloat16().to(dev)
        y = RowShardedLinear(qw, sc, su, sv, device=dev)(x)
        full = ops.linear(x, qw.to(dev), sc.to(dev), su.to(dev), sv.to(dev))
        ok = bool(torch.equal(y, full))
        # the same through peer stores from the kernel epilogue (symmetric memory, no collective kernel), three calls in a row
        peer = RowShardedLinear(qw, sc, su, sv, device=dev, gather="peer")
        for i in range(3):
            xi = (x * (i + 1)).contiguous()
            want = ops.linear(xi, qw.to(dev), sc.to(dev), su.to(dev), sv.to(dev))
            ok = ok and bool(torch.equal(peer(xi), want))
        # expert-parallel MoE, 8 experts over the two ranks: device-routed grouped launches (pairs of the other rank's experts are
        # skipped by the kernel) against host routing and against the CPU reference
        from htr_b200.sharded import ExpertParallelMoE

        experts, xm, ids, w = _moe_inputs(E=8, h=256, inter=128, T=6, k=2, K=3, seed=4)
        moe = ExpertParallelMoE(experts, device=dev)
        y_grp = moe(xm.to(dev), ids, w).float().cpu()
        y_loop = moe(xm.to(dev), ids, w, grouped=False).float().cpu()
        want = _moe_reference(experts, xm, ids, w, _oracle_linear())
        ok = ok and float((y_grp - want).norm() / want.norm()) <= 1e-5 and float((y_loop - want).norm() / want.norm()) <= 1e-5
        torch.cuda.synchronize()
        q.put((rank, ok, tuple(y.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_two_nccl_ranks_match_single_gpu_bit_for_bit():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ok and shape == (3, 128 * 11) for _, ok, shape in res)
