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
        full_w = [t.to(dev) for t in (qw, sc, su, sv)]
        x = torch.randn(2, 1024, generator=torch.Generator().manual_seed(9)).bfloat16().to(dev)
        # up to two rows run on the integer-exact kernel, whose sums do not depend on the launch decomposition: the gathered result
        # is the single-GPU result (under the same flag) bit for bit
        y = RowShardedLinear(qw, sc, su, sv, device=dev)(x)
        with ops.exact_sums():
            full = ops.linear(x, *full_w)
        ok = bool(torch.equal(y, full))
        # the same through peer stores from the kernel epilogue (symmetric memory, delivery flags, no collective kernel), three
        # calls in a row, one and two rows
        from htr_b200 import sharded as sharded_mod

        peer = RowShardedLinear(qw, sc, su, sv, device=dev, gather="peer")
        for order in ("kernel", "barrier", "flags"):                         # the three ways of ordering the ranks after the peer stores
            sharded_mod.PEER_ORDER = order
            for i in range(3):
                xi = (x[:1 + i % 2] * (i + 1)).contiguous()
                with ops.exact_sums():
                    want = ops.linear(xi, *full_w)
                ok = ok and bool(torch.equal(peer(xi), want))
        peer.peer.check()                                                    # no bounded wait ran out
        sharded_mod.PEER_ORDER = "kernel"
        # three rows (float32 sums per window): within bf16 rounding of the single-GPU result; eight and twenty rows: the tensor-core
        # GEMM with the peer-store epilogue; forty rows: local GEMM + all-gather
        for rows in (3, 8, 20, 40):
            xr = torch.randn(rows, 1024, generator=torch.Generator().manual_seed(rows)).bfloat16().to(dev)
            got, want = peer(xr).float(), ops.linear(xr, *full_w).float()
            ok = ok and float((got - want).norm() / want.norm()) <= 4e-3
        # expert-parallel MoE, 8 experts over the two ranks: device-routed grouped launches (pairs of the other rank's experts are
        # skipped by the kernel) against host routing and against the CPU reference
        from htr_b200.sharded import ExpertParallelMoE

        experts, xm, ids, w = _moe_inputs(E=8, h=256, inter=128, T=6, k=2, K=3, seed=4)
        moe = ExpertParallelMoE(experts, device=dev)
        y_grp = moe(xm.to(dev), ids, w).float().cpu()
        y_loop = moe(xm.to(dev), ids, w, grouped=False).float().cpu()
        want = _moe_reference(experts, xm, ids, w, _oracle_linear())
        ok = ok and float((y_grp - want).norm() / want.norm()) <= 1e-5 and float((y_loop - want).norm() / want.norm()) <= 1e-5
        # the default combine across ranks ("rows": the down launch stores each pair's row into every rank, one barrier, the same
        # weighted sum as on one GPU) equals a one-rank layer that holds all experts, bit for bit; three calls in a row (the two
        # halves of the exchange matrix alternate), float32 and bf16
        solo = None
        for r in range(world):                                               # every rank creates every group, as torch.distributed requires
            g = dist.new_group([r])
            solo = g if r == rank else solo
        one = ExpertParallelMoE(experts, device=dev, group=solo)
        moe.plan_for_share = False                                           # the single-GPU launch plan: bit for bit
        for xin in (xm, xm.bfloat16(), xm * 2):
            ok = ok and bool(torch.equal(moe(xin.to(dev), ids, w), one(xin.to(dev), ids, w)))
        moe.plan_for_share = True                                            # the default: more thread blocks per owned pair,
        y_rows = moe(xm.to(dev), ids, w)
        for xin in (xm, xm.bfloat16()):                                      # float32 partial sums in another order
            a, b = moe(xin.to(dev), ids, w).float(), one(xin.to(dev), ids, w).float()
            ok = ok and float((a - b).norm() / b.norm()) <= (1e-6 if xin.dtype == torch.float32 else 4e-3)
            g = [torch.empty_like(a) for _ in range(world)]
            dist.all_gather(g, a)
            ok = ok and all(bool(torch.equal(t, a)) for t in g)             # every rank holds the same bits
        # the other two combines (float32 partial sums by peer stores, or by all-gather; rank-ordered add) agree to rounding
        y_nccl = moe(xm.to(dev), ids, w, combine="nccl").float().cpu()
        ok = ok and float((y_grp - y_nccl).norm() / y_nccl.norm()) <= 1e-6
        y_peer = moe(xm.to(dev), ids, w, combine="peer").float().cpu()
        ok = ok and float((y_peer - y_nccl).norm() / y_nccl.norm()) <= 1e-6
        for order in ("barrier", "flags", "barrier"):
            sharded_mod.PEER_ORDER = order
            ok = ok and bool(torch.equal(moe(xm.to(dev), ids, w, combine="peer").float().cpu(), y_peer))
        sharded_mod.PEER_ORDER = "barrier"                                   # the row exchange under torch's barrier as well
        ok = ok and bool(torch.equal(moe(xm.to(dev), ids, w), y_rows))
        sharded_mod.PEER_ORDER = "kernel"
        for ex in moe._rows.values():
            ex["barrier"].check()
        ok = ok and int(moe._peer["status"].item()) == 0
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
    assert all(ok and shape == (2, 128 * 11) for _, ok, shape in res)


@pytest.mark.gpu
def test_peer_barrier_gives_up_and_reports_the_missing_rank():
    """The library's cross-rank barrier kernel waits with a bound: emulated on one GPU as rank 0 of two, with a peer whose word
    nothing raises, it returns after about two seconds, sets the missing rank's bit and leaves the context usable; once the
    peer's word is there the next barrier passes at once."""
    from htr_b200 import ops

    dev = torch.device("cuda:0")
    flags = torch.zeros(64, dtype=torch.int32, device=dev)                  # this GPU's words: word 0 = rank 0 (itself), word 1 = rank 1
    elsewhere = torch.zeros(64, dtype=torch.int32, device=dev)              # stands for rank 1's flag array
    words = torch.tensor([flags.data_ptr(), elsewhere.data_ptr()], dtype=torch.int64, device=dev)
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.peer_barrier(words, flags, epoch, 2, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0b10 and int(epoch.item()) == 1
    assert int(flags[0].item()) == 1 and int(elsewhere[0].item()) == 1      # its own word was raised in both arrays
    flags[1] = 2                                                            # rank 1 arrives at barrier 2
    status.zero_()
    ops.peer_barrier(words, flags, epoch, 2, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(epoch.item()) == 2
    assert float(torch.ones(4, device=dev).sum()) == 4.0                    # the device still answers


@pytest.mark.gpu
def test_peer_wait_gives_up_and_reports_the_missing_rank():
    """The consumer's wait for delivery flags is bounded: with a flag that nothing raises, the kernel returns after about two
    seconds, sets the missing rank's bit in the status word and leaves the context usable."""
    from htr_b200 import ops

    dev = torch.device("cuda:0")
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    flags[0] = 1                                                            # rank 0 has delivered, rank 1 never does
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.peer_wait(flags, epoch, 2, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0b10 and int(epoch.item()) == 1
    flags[1] = 2                                                            # both ranks are at call 2 now: the next wait passes at once
    flags[0] = 2
    status.zero_()
    ops.peer_wait(flags, epoch, 2, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(epoch.item()) == 2
    assert float(torch.ones(4, device=dev).sum()) == 4.0                    # the device still answers


def _failing_gloo_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from htr_b200.sharded import all_gather_rows

        y = torch.full((2, 4), float(rank))
        all_gather_rows(y)                                                   # one healthy round first
        if rank == 1:
            raise RuntimeError("injected failure: this rank leaves before the collective")
        try:
            all_gather_rows(y)                                               # the peer never joins: must end with an error, not hang
            q.put((rank, "returned"))
        except Exception as e:                                               # noqa: BLE001 - any error from the backend will do
            q.put((rank, "error: " + type(e).__name__))
    except RuntimeError as e:
        q.put((rank, "left: " + str(e)[:40]))
        q.close()
        q.join_thread()                                                      # the message is on its way before the process dies
        os._exit(3)                                                          # leave without tearing the group down, as a crashed rank does
    finally:
        if rank == 0:
            try:
                dist.destroy_process_group()
            except Exception:                                                # noqa: BLE001
                pass


def test_a_rank_that_leaves_ends_the_others_collective_with_an_error():
    """Host-side failure handling of the sharded forms: the gathers are torch.distributed collectives, so a rank that dies
    between steps surfaces on its peers as an exception from the next collective within the process group's timeout (20 s
    here) -- never as a hang.  Two gloo ranks on CPU; rank 1 raises before the second all-gather."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=90) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert got[1].startswith("left")
    assert got[0].startswith("error"), got
    assert procs[1].exitcode == 3
