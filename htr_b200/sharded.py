"""Multi-GPU execution of packed linears on one NVLink box: one process per GPU over torch.distributed.

The reference runs on one device only (tensor parallelism is refused, htr/vllm_plugin.py:91).  What makes sharding
natural is stated in its LM-head tool (htr/lmhead.py:9-11) and its format text (docs/FORMAT.md:31-32): output rows are
independent at the granularity of a 128-row block (row scales per row, `sv` per 8 rows, qweight per 16 rows, output
Hadamard per 128 rows), and fused modules simply concatenate along the output dimension.

* RowShardedLinear   a tall linear (LM head, MLP up-projection) cut into contiguous runs of 128-row blocks, one run per
                     rank; `x` and `su` are replicated; the bf16 outputs are all-gathered (NCCL over NVLink).  The gathered
                     result equals the single-GPU result bit for bit, because a row block is computed by the same code
                     whichever rank owns it.
* ExpertParallelMoE  a SwiGLU mixture-of-experts layer whose experts are dealt to the ranks in contiguous groups; tokens
                     and routing are replicated; every rank evaluates its experts for the tokens routed to them and the
                     partial outputs are combined by all-gather + addition in rank order (deterministic).

`linear_fn` is injectable so that the host-side logic (partitioning, padding, gather layout, routing) can be exercised on CPU
ranks with the gloo backend; the default is the CUDA operator, which has no CPU path.
"""
import torch
import torch.distributed as dist


# How the ranks order themselves after peer stores:
#   "kernel"  = the producer kernel ends, then htr_peer_barrier: one small kernel per rank that becomes resident behind the producer,
#               raises this rank's word in every rank's flag array and waits (bounded) for every rank's word here;
#   "barrier" = the same with the barrier kernel of torch's symmetric memory;
#   "flags"   = the producer kernel raises the delivery flags itself (its last thread block) and the consumer runs a bounded wait
#               (htr_peer_wait).
PEER_ORDER = "kernel"


def row_block_partition(m, world):
    """Split m/128 row blocks into `world` contiguous runs of equal padded length.
    Returns (blocks_per_rank, [(first_block, real_blocks), ...]).  151936 rows = 1187 blocks over 8 ranks -> 149 per rank,
    the last rank holds 144 real blocks and 5 padding blocks."""
    if m % 128:
        raise ValueError("row sharding needs m % 128 == 0")
    blocks = m // 128
    per = -(-blocks // world)
    runs = []
    for r in range(world):
        first = min(r * per, blocks)
        runs.append((first, max(0, min(per, blocks - first))))
    return per, runs


def _pad_rows(t, rows):
    if t.shape[0] == rows:
        return t.contiguous()
    pad = torch.zeros((rows - t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    return torch.cat([t, pad]).contiguous()


def shard_rows(qweight, scales, sv, bias, world, rank):
    """The rank's run of row blocks of a packed linear, zero-padded to the common length (a zero scale makes a padding
    row produce exactly 0).  Units: qweight strips of 16 rows, scales per row, sv bytes per 8 rows."""
    m = qweight.shape[0] * 16
    per, runs = row_block_partition(m, world)
    first, real = runs[rank]
    lo, hi = first * 128, (first + real) * 128
    q = _pad_rows(qweight[lo // 16:hi // 16], per * 8)
    s = _pad_rows(scales[lo:hi], per * 128)
    v = _pad_rows(sv[lo // 8:hi // 8], per * 16)
    b = None if bias is None else _pad_rows(bias[lo:hi], per * 128)
    return q, s, v, b


def _default_linear():
    from . import ops

    return ops.linear


def _world(group):
    if not dist.is_available() or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def all_gather_rows(y_local, group=None):
    """[M, r] on every rank -> [world, M, r] (one collective; NCCL gathers into one tensor, gloo into a list)."""
    world, _ = _world(group)
    if world == 1:
        return y_local.unsqueeze(0)
    y_local = y_local.contiguous()
    if dist.get_backend(group) == "nccl":
        out = torch.empty((world,) + tuple(y_local.shape), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(out, y_local, group=group)
        return out
    parts = [torch.empty_like(y_local) for _ in range(world)]
    dist.all_gather(parts, y_local, group=group)
    return torch.stack(parts)


class RankBarrier:
    """Barrier across the ranks of one NVLink box as one small kernel per rank (htr_peer_barrier): flag words in symmetric memory,
    word r of a rank's array is raised by rank r; the count of barriers passed lives in device memory (CUDA-graph replay keeps it)."""

    def __init__(self, world, rank, device, group=None):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # plain peer stores and atomics only
        import torch.distributed._symmetric_memory as symm_mem

        grp = group if group is not None else dist.group.WORLD
        self.world = world
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.hdl = symm_mem.rendezvous(self.flags, grp)
        self.peer_words = torch.tensor([int(p) + 4 * rank for p in self.hdl.buffer_ptrs], dtype=torch.int64, device=device)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)              # bit r: rank r did not arrive in time
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)                                                      # every rank's words are zero before anyone signals

    def __call__(self):
        from . import ops

        ops.peer_barrier(self.peer_words, self.flags, self.epoch, self.world, self.status)

    def check(self):
        """Host-side check (synchronises): raises if a bounded wait ran out since the last check."""
        missed = int(self.status.item())
        if missed:
            self.status.zero_()
            raise RuntimeError(f"cross-rank barrier timed out waiting for ranks {[r for r in range(self.world) if missed >> r & 1]}")


class PeerGather:
    """Gather buffers in symmetric memory: every rank maps every rank's buffer, so a kernel can store its output rows
    straight into all of them over NVLink (htr_linear_peers) and no collective kernel runs.  The ranks then order themselves
    with `barrier()` (one small kernel across the ranks) or, with delivery flags (htr_linear_peers_signal: the producer kernel
    raises this rank's word in every rank's flag array), with `wait()`, a bounded wait on the current stream.

    Two alternating buffers: a rank that is one call ahead writes the half that its peers have finished reading (a rank consumes
    the result of call i - 1, on its stream, before it launches call i + 1).  A CUDA graph that is replayed back to back must
    therefore capture an even number of calls (both halves), or end with a barrier of its own."""

    def __init__(self, world, rank, max_rows, rows_per_rank, dtype, device, group=None):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # plain peer stores only, no NVLink multicast objects
        import torch.distributed._symmetric_memory as symm_mem

        grp = group if group is not None else dist.group.WORLD
        self.world, self.rank, self.max_rows, self.rows_per_rank = world, rank, max_rows, rows_per_rank
        self.buf = symm_mem.empty((2, world, max_rows, rows_per_rank), dtype=dtype, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, grp)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=device)          # word r: deliveries of rank r into this GPU's buffer
        self.flags.zero_()
        self.flag_hdl = symm_mem.rendezvous(self.flags, grp)
        self.flag_ptrs = [int(p) + 4 * rank for p in self.flag_hdl.buffer_ptrs]     # this rank's word in every rank's array
        self.rank_barrier = RankBarrier(world, rank, device, group)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)              # bit r: rank r missed a bounded wait
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)                                                      # every rank's flags are zero before anyone signals
        self.flip = 0
        self.esize = self.buf.element_size()

    def target(self):
        """(peer addresses of the buffer half in use, element offset of this rank's block inside it)"""
        half = self.flip * self.world * self.max_rows * self.rows_per_rank
        return [p + half * self.esize for p in self.ptrs], self.rank * self.max_rows * self.rows_per_rank

    def wait(self, count=1):
        from . import ops

        ops.peer_wait(self.flags, self.epoch, self.world, self.status, count)

    def barrier(self):
        """Order the ranks after peer stores that carried no delivery signal (PEER_ORDER "kernel" or "barrier")."""
        if PEER_ORDER == "barrier":
            self.hdl.barrier(channel=0)
        else:
            self.rank_barrier()

    def check(self):
        """Host-side check (synchronises): raises if a bounded wait ran out since the last check."""
        missed = int(self.status.item())
        if missed:
            self.status.zero_()
            raise RuntimeError(f"peer delivery wait timed out for ranks {[r for r in range(self.world) if missed >> r & 1]}")
        self.rank_barrier.check()

    def result(self, rows):
        out = self.buf[self.flip, :, :rows, :]
        self.flip ^= 1
        return out


class RowShardedLinear:
    """y = x @ W^T (+bias) with W's rows dealt to the ranks of `group`; every rank gets the full [.., m] result.

    gather="nccl": all-gather of the local outputs.  gather="peer": the kernel's epilogue stores its rows into every rank's
    gather buffer itself (the GEMV up to 4 activation rows, the tensor-core GEMM up to 32) and one barrier kernel orders the ranks;
    larger batches run the GEMM locally and all-gather its output."""

    def __init__(self, qweight, scales, su, sv, bias=None, group=None, device=None, linear_fn=None, gather="nccl", dtype=torch.bfloat16):
        self.group = group
        self.world, self.rank = _world(group)
        self.m = qweight.shape[0] * 16
        self.n = qweight.shape[1] * 16
        q, s, v, b = shard_rows(qweight, scales, sv, bias, self.world, self.rank)
        dev = device if device is not None else qweight.device
        self.qweight, self.scales, self.sv = q.to(dev), s.to(dev), v.to(dev)
        self.su = su.to(dev).contiguous()
        self.bias = None if b is None else b.to(dev)
        self._cuda_operator = linear_fn is None
        self.linear_fn = linear_fn or _default_linear()
        self.peer = None
        if gather == "peer" and self.world > 1:
            self.peer = PeerGather(self.world, self.rank, 32, self.qweight.shape[0] * 16, dtype, dev, group)

    def _exact(self):
        """Row shards must reproduce the unsharded rows whatever the shard count: up to four rows run on the integer-exact kernel."""
        if self._cuda_operator:
            from . import ops

            return ops.exact_sums()
        import contextlib

        return contextlib.nullcontext()

    def local(self, x):
        """This rank's slice of the output, [.., rows_per_rank] (padding rows are zero)."""
        bias = None if self.bias is None else self.bias.to(x.dtype)
        with self._exact():
            return self.linear_fn(x, self.qweight, self.scales, self.su, self.sv, bias)

    def __call__(self, x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.n)
        if self.peer is not None and 1 <= x2.shape[0] <= 4 and x2.dtype == self.peer.buf.dtype:
            from . import ops

            ptrs, off = self.peer.target()
            bias = None if self.bias is None else self.bias.to(x2.dtype)
            flags = PEER_ORDER == "flags"
            with ops.exact_sums():
                ops.linear_into_peers(x2.contiguous(), self.qweight, self.scales, self.su, self.sv, bias, ptrs, off,
                                      self.peer.flag_ptrs if flags else None)
            if flags:
                self.peer.wait()
            else:
                self.peer.barrier()
            g = self.peer.result(x2.shape[0])                                # [world, M, rows_per_rank]
            rows = x2.shape[0]
        elif self.peer is not None and 4 < x2.shape[0] <= self.peer.max_rows and x2.dtype == self.peer.buf.dtype:
            # the tensor-core GEMM's epilogue stores into every rank's gather buffer as well; one barrier orders the ranks
            from . import ops

            ptrs, off = self.peer.target()
            bias = None if self.bias is None else self.bias.to(x2.dtype)
            ops.gemm_into_peers(x2.contiguous(), self.qweight, self.scales, self.su, self.sv, bias, ptrs, off)
            self.peer.barrier()
            g = self.peer.result(x2.shape[0])
            rows = x2.shape[0]
        else:
            y = self.local(x2)
            g = all_gather_rows(y, self.group)                               # [world, M, rows_per_rank]
            rows = y.shape[0]
        full = g.permute(1, 0, 2).reshape(rows, -1)[:, :self.m]
        return full.reshape(*lead, self.m)


def expert_partition(num_experts, world):
    """Contiguous groups of experts per rank: [(first, count), ...]."""
    per = -(-num_experts // world)
    return [(min(r * per, num_experts), max(0, min(per, num_experts - r * per))) for r in range(world)]


class ExpertParallelMoE:
    """SwiGLU mixture of experts, y_t = sum_k gate[t,k] * down_e( silu(gate_e(x_t)) * up_e(x_t) ), e = ids[t,k].

    `experts[e]` = dict(gate_up=(qweight, scales, su, sv), down=(qweight, scales, su, sv)); gate_up is the fused
    [2*I, h] matrix (gate rows first, as the reference's encoder groups gate and up under one `su`,
    htr/moe_encode.py:181-196).  Only this rank's experts are kept."""

    def __init__(self, experts, group=None, device=None, linear_fn=None):
        self.group = group
        self.world, self.rank = _world(group)
        self.num_experts = len(experts)
        first, count = expert_partition(self.num_experts, self.world)[self.rank]
        self.first, self.count = first, count
        dev = device

        def put(t):
            return tuple(a.to(dev).contiguous() if dev is not None else a.contiguous() for a in t)

        self.local = {e: dict(gate_up=put(experts[e]["gate_up"]), down=put(experts[e]["down"])) for e in range(first, first + count)}
        self.linear_fn = linear_fn or _default_linear()
        self._tables = None
        self._peer = None
        self._rows = {}
        # Plan the routed launches for the share of the pairs whose expert lives here (world times more thread blocks than the GPU
        # holds; those of the other ranks' pairs leave at once).  The float32 partial sums of a row then add up in another order
        # than on one GPU: every rank still holds the same bits (a row is computed once, by its owner), equal to the single-GPU
        # layer to float32 rounding.  False keeps the single-GPU plan and with it equality with the single-GPU layer bit for bit.
        self.plan_for_share = True

    def _address_tables(self, dev):
        """int64 device tensors [all experts] with the addresses of each expert's wire tensors (for the grouped kernel);
        experts of other ranks have address 0, which the kernel skips."""
        if self._tables is None:
            def col(which, i):
                return torch.tensor([self.local[e][which][i].data_ptr() if e in self.local else 0 for e in range(self.num_experts)],
                                    dtype=torch.int64, device=dev)
            self._tables = {w: tuple(col(w, i) for i in range(4)) for w in ("gate_up", "down")}
        return self._tables

    def _row_exchange(self, pairs, hdim, dtype, dev):
        """Symmetric-memory matrices [2 halves][pairs][h] that every rank maps: a routed launch stores the output row of each pair
        this rank owns into all of them.  Two halves alternate (a rank one call ahead writes the half its peers have finished
        reading: it passed the barrier of the call before, which its peers reach only after they have consumed the call before that;
        a CUDA graph replayed back to back must capture an even number of calls)."""
        key = (dtype, hdim)
        ex = self._rows.get(key)
        if ex is None or ex["pairs"] < pairs:
            import os

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
            import torch.distributed._symmetric_memory as symm_mem

            grp = self.group if self.group is not None else dist.group.WORLD
            cap = max(512, pairs)
            buf = symm_mem.empty((2, cap, hdim), dtype=dtype, device=dev)
            hdl = symm_mem.rendezvous(buf, grp)
            half_bytes = cap * hdim * buf.element_size()
            ptrs = [[int(p) + hf * half_bytes for p in hdl.buffer_ptrs] for hf in (0, 1)]
            ex = dict(pairs=cap, buf=buf, hdl=hdl, ptrs=ptrs, flip=0, barrier=RankBarrier(self.world, self.rank, dev, self.group))
            torch.cuda.synchronize(dev)
            dist.barrier(group=grp)
            self._rows[key] = ex
        return ex

    def routed_outputs(self, x, topk_ids, exchange=False):
        """Expert outputs of every (token, slot) pair, [T * k, h] in x.dtype, with two routed launches over all pairs: gate_up reads
        token row pair // k, down reads the pair's [gate | up] row and applies SwiGLU while staging it (bf16; other dtypes use a
        separate activation step).  Routing stays on the device (no host round trip, capturable in a CUDA graph); pairs routed to
        another rank's experts are skipped by the kernel (null weight address).  Without `exchange` their rows stay zero; with it
        the down launch stores each row into every rank's matrix (htr_linear_routed_peers) and, after one barrier across the ranks,
        every rank holds the rows of all pairs, each computed by the rank that owns its expert."""
        from . import _lib, ops

        T, hdim = x.shape
        k = topk_ids.shape[1]
        dev = x.device
        tabs = self._address_tables(dev)
        route = topk_ids.to(device=dev, dtype=torch.int64).reshape(-1).contiguous()
        any_e = next(iter(self.local.values()))
        mt_gu, nt_gu, W = any_e["gate_up"][0].shape
        mt_dn, nt_dn, _ = any_e["down"][0].shape
        K = W // 8
        x = x.contiguous()
        skip = self.world > 1 and not exchange                          # rows of skipped pairs must read as zero
        alloc = torch.zeros if skip else torch.empty
        # (with `exchange`, the gate_up rows of pairs owned elsewhere are never read: the down launch skips the same pairs)
        share = self.world if (x.is_cuda and self.plan_for_share) else 1  # one pair in `world` has its expert here
        gu = ops.linear_routed(x, route, tabs["gate_up"], mt_gu, nt_gu, K, x_div=k, out=alloc(T * k, mt_gu * 16, dtype=x.dtype, device=dev),
                               share=share)
        if x.dtype == torch.bfloat16:
            act, prologue = gu, ops.PROLOGUE_SWIGLU
        else:
            inter = mt_gu * 8
            act, prologue = (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]).contiguous(), ops.PROLOGUE_NONE
        if not exchange:
            return ops.linear_routed(act, route, tabs["down"], mt_dn, nt_dn, K, prologue=prologue, out=alloc(T * k, mt_dn * 16, dtype=x.dtype, device=dev),
                                     share=share)
        ex = self._row_exchange(T * k, mt_dn * 16, x.dtype, dev)
        half = ex["flip"]
        ex["flip"] ^= 1
        dn = ex["buf"][half, :T * k]
        ops.linear_routed(act, route, tabs["down"], mt_dn, nt_dn, K, prologue=prologue, out=dn, peer_ptrs=ex["ptrs"][half], share=share)
        if PEER_ORDER == "barrier":
            ex["hdl"].barrier(channel=0)
        else:
            ex["barrier"]()
        return dn

    @staticmethod
    def weighted_sum(dn, topk_w, T, k):
        """y[t] = sum_j w[t, j] * dn[t * k + j] (htr_moe_weighted_sum: float32 sums in slot order, one rounding)."""
        from . import _lib

        dev = dn.device
        gates = topk_w.to(device=dev, dtype=torch.float32).contiguous()
        out = torch.empty(T, dn.shape[1], dtype=dn.dtype, device=dev)
        code = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}[dn.dtype]
        with torch.cuda.device(dev):
            rc = _lib.lib.htr_moe_weighted_sum(dn.data_ptr(), code, gates.data_ptr(), T, k, dn.shape[1], out.data_ptr(),
                                               torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(rc, "htr_moe_weighted_sum")
        return out

    def partial_grouped(self, x, topk_ids, topk_w):
        """Contribution of this rank's experts, float32 [T, h]: the routed launches + the gate-weighted sum over the slots."""
        T, k = topk_ids.shape
        dn = self.routed_outputs(x, topk_ids)
        return torch.einsum("tkh,tk->th", dn.view(T, k, -1).float(), topk_w.to(device=x.device, dtype=torch.float32))

    def _peer_combine(self, dn, topk_w, T, k, hdim, dtype):
        """Combine over the ranks without a collective: the gate-weighted sum of this rank's pairs is stored into every rank's
        buffer (htr_moe_combine_peers: plain peer stores), the ranks order themselves (PEER_ORDER) and every rank adds the parts in
        rank order (htr_rank_sum), so all ranks hold the same bits."""
        from . import _lib, ops

        dev = dn.device
        pc = self._peer
        if pc is None:
            import os

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem

            grp = self.group if self.group is not None else dist.group.WORLD
            pc = {"max_t": 64}
            pc["buf"] = symm_mem.empty((2, self.world, pc["max_t"], hdim), dtype=torch.float32, device=dev)
            hdl = symm_mem.rendezvous(pc["buf"], grp)
            pc["flags"] = symm_mem.empty(64, dtype=torch.int32, device=dev)
            pc["flags"].zero_()
            fh = symm_mem.rendezvous(pc["flags"], grp)
            pc["hdls"] = (hdl, fh)
            half_bytes = self.world * pc["max_t"] * hdim * 4
            pc["out_ptrs"] = [torch.tensor([int(p) + hf * half_bytes for p in hdl.buffer_ptrs], dtype=torch.int64, device=dev) for hf in (0, 1)]
            pc["flag_ptrs"] = torch.tensor([int(p) + 4 * self.rank for p in fh.buffer_ptrs], dtype=torch.int64, device=dev)
            pc["epoch"] = torch.zeros(1, dtype=torch.int32, device=dev)
            pc["status"] = torch.zeros(1, dtype=torch.int32, device=dev)
            pc["done"] = torch.zeros(1, dtype=torch.int32, device=dev)
            pc["flip"] = 0
            torch.cuda.synchronize(dev)
            dist.barrier(group=grp)
            self._peer = pc
        half = pc["flip"]
        pc["flip"] ^= 1
        st = torch.cuda.current_stream(dev).cuda_stream
        code = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}[dtype]
        gates = topk_w.to(device=dev, dtype=torch.float32).contiguous()
        flags = PEER_ORDER == "flags"
        rc = _lib.lib.htr_moe_combine_peers(dn.data_ptr(), code, gates.data_ptr(), T, k, hdim, pc["out_ptrs"][half].data_ptr(), self.world,
                                            self.rank * pc["max_t"] * hdim, pc["flag_ptrs"].data_ptr() if flags else None,
                                            pc["done"].data_ptr() if flags else None, st)
        _lib.check(rc, "htr_moe_combine_peers")
        if flags:
            ops.peer_wait(pc["flags"], pc["epoch"], self.world, pc["status"])
        else:
            pc["hdls"][0].barrier(channel=0)
        out = torch.empty(T, hdim, dtype=dtype, device=dev)
        rc = _lib.lib.htr_rank_sum(pc["buf"][half].data_ptr(), self.world, pc["max_t"] * hdim, T, hdim, out.data_ptr(), code, st)
        _lib.check(rc, "htr_rank_sum")
        return out

    def partial(self, x, topk_ids, topk_w):
        """Contribution of this rank's experts, float32 [T, h].  Routing is resolved on the host."""
        T, hdim = x.shape
        out = torch.zeros(T, hdim, dtype=torch.float32, device=x.device)
        ids = topk_ids.detach().cpu()
        for e in range(self.first, self.first + self.count):                 # fixed expert order: deterministic sums
            hit = (ids == e).nonzero(as_tuple=False)
            if hit.numel() == 0:
                continue
            tok = hit[:, 0].to(x.device)
            w = topk_w[hit[:, 0], hit[:, 1]].to(device=x.device, dtype=torch.float32)
            gu = self.linear_fn(x.index_select(0, tok), *self.local[e]["gate_up"])
            inter = gu.shape[1] // 2
            act = (torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()).to(x.dtype)
            d = self.linear_fn(act, *self.local[e]["down"])
            out.index_add_(0, tok, d.float() * w[:, None])
        return out

    def __call__(self, x, topk_ids, topk_w, grouped=None, combine=None):
        """combine (several ranks, CUDA, grouped form, NCCL group; default "rows" where it applies):
        "rows" = the down launch stores each pair's row into every rank, one barrier, then the same weighted sum as on one GPU
                 (every rank holds the same bits; with plan_for_share = False they equal the single-GPU result bit for bit; up to
                 4096 pairs);
        "peer" = peer stores of the ranks' float32 partial sums + rank-ordered add (up to 64 tokens);
        "nccl" = all-gather of the float32 parts + rank-ordered add."""
        use_grouped = (x.is_cuda and self.count > 0) if grouped is None else grouped
        T, hdim = x.shape
        k = topk_ids.shape[1]
        if self.world == 1 and use_grouped and x.is_cuda:
            return self.weighted_sum(self.routed_outputs(x, topk_ids), topk_w, T, k)
        peers_ok = (self.world > 1 and use_grouped and x.is_cuda and self.num_experts >= self.world and dist.get_backend(self.group) == "nccl")
        if peers_ok and combine in (None, "rows") and T * k <= 4096:
            return self.weighted_sum(self.routed_outputs(x, topk_ids, exchange=True), topk_w, T, k)
        if peers_ok and combine in (None, "peer") and T <= 64:
            dn = self.routed_outputs(x, topk_ids)
            return self._peer_combine(dn, topk_w, T, k, hdim, x.dtype)
        part = self.partial_grouped(x, topk_ids, topk_w) if use_grouped else self.partial(x, topk_ids, topk_w)
        if self.world == 1:
            return part.to(x.dtype)
        g = all_gather_rows(part, self.group)                                # [world, T, h] float32
        total = g[0].clone()
        for r in range(1, self.world):                                       # rank order: every rank adds identically
            total += g[r]
        return total.to(x.dtype)
