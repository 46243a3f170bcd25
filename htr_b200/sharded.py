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


class PeerGather:
    """Gather buffers in symmetric memory: every rank maps every rank's buffer, so a kernel can store its output rows
    straight into all of them over NVLink (htr_linear_peers) and no collective kernel runs.  `barrier()` orders the
    ranks on the current stream: after it, every rank's rows are in this rank's buffer.

    Two alternating buffers let a fast rank start the next call while a slow one still reads the previous result."""

    def __init__(self, world, rank, max_rows, rows_per_rank, dtype, device, group=None):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # plain peer stores only, no NVLink multicast objects
        import torch.distributed._symmetric_memory as symm_mem

        self.world, self.rank, self.max_rows, self.rows_per_rank = world, rank, max_rows, rows_per_rank
        self.buf = symm_mem.empty((2, world, max_rows, rows_per_rank), dtype=dtype, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.flip = 0
        self.esize = self.buf.element_size()

    def target(self):
        """(peer addresses of the buffer half in use, element offset of this rank's block inside it)"""
        half = self.flip * self.world * self.max_rows * self.rows_per_rank
        return [p + half * self.esize for p in self.ptrs], self.rank * self.max_rows * self.rows_per_rank

    def barrier(self):
        self.hdl.barrier(channel=0)

    def result(self, rows):
        out = self.buf[self.flip, :, :rows, :]
        self.flip ^= 1
        return out


class RowShardedLinear:
    """y = x @ W^T (+bias) with W's rows dealt to the ranks of `group`; every rank gets the full [.., m] result.

    gather="nccl": all-gather of the local outputs.  gather="peer": the GEMV's epilogue stores its rows into every rank's
    gather buffer itself (up to 8 activation rows; larger batches fall back to the all-gather)."""

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
        self.linear_fn = linear_fn or _default_linear()
        self.peer = None
        if gather == "peer" and self.world > 1:
            self.peer = PeerGather(self.world, self.rank, 8, self.qweight.shape[0] * 16, dtype, dev, group)

    def local(self, x):
        """This rank's slice of the output, [.., rows_per_rank] (padding rows are zero)."""
        bias = None if self.bias is None else self.bias.to(x.dtype)
        return self.linear_fn(x, self.qweight, self.scales, self.su, self.sv, bias)

    def __call__(self, x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.n)
        if self.peer is not None and 1 <= x2.shape[0] <= 8 and x2.dtype == self.peer.buf.dtype:
            from . import ops

            ptrs, off = self.peer.target()
            bias = None if self.bias is None else self.bias.to(x2.dtype)
            ops.linear_into_peers(x2.contiguous(), self.qweight, self.scales, self.su, self.sv, bias, ptrs, off)
            self.peer.barrier()
            g = self.peer.result(x2.shape[0])                                # [world, M, rows_per_rank]
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

    def _address_tables(self, dev):
        """int64 device tensors [all experts] with the addresses of each expert's wire tensors (for the grouped kernel);
        experts of other ranks have address 0, which the kernel skips."""
        if self._tables is None:
            def col(which, i):
                return torch.tensor([self.local[e][which][i].data_ptr() if e in self.local else 0 for e in range(self.num_experts)],
                                    dtype=torch.int64, device=dev)
            self._tables = {w: tuple(col(w, i) for i in range(4)) for w in ("gate_up", "down")}
        return self._tables

    def partial_grouped(self, x, topk_ids, topk_w):
        """The same contribution with two routed launches over all (token, slot) pairs: gate_up reads token row pair // k, down
        reads the pair's [gate | up] row and applies SwiGLU while staging it (bf16; other dtypes use a separate activation step).
        Routing stays on the device (no host round trip, capturable in a CUDA graph); pairs routed to another rank's experts are
        skipped by the kernel (null weight address) and contribute zero here."""
        from . import ops

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
        skip = self.world > 1                                            # rows of skipped pairs must read as zero
        alloc = torch.zeros if skip else torch.empty
        gu = ops.linear_routed(x, route, tabs["gate_up"], mt_gu, nt_gu, K, x_div=k, out=alloc(T * k, mt_gu * 16, dtype=x.dtype, device=dev))
        dn = alloc(T * k, mt_dn * 16, dtype=x.dtype, device=dev)
        if x.dtype == torch.bfloat16:
            ops.linear_routed(gu, route, tabs["down"], mt_dn, nt_dn, K, prologue=ops.PROLOGUE_SWIGLU, out=dn)
        else:
            inter = mt_gu * 8
            act = (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]).contiguous()
            ops.linear_routed(act, route, tabs["down"], mt_dn, nt_dn, K, out=dn)
        return torch.einsum("tkh,tk->th", dn.view(T, k, -1).float(), topk_w.to(device=dev, dtype=torch.float32))

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

    def __call__(self, x, topk_ids, topk_w, grouped=None):
        use_grouped = (x.is_cuda and self.count > 0) if grouped is None else grouped
        part = self.partial_grouped(x, topk_ids, topk_w) if use_grouped else self.partial(x, topk_ids, topk_w)
        if self.world == 1:
            return part.to(x.dtype)
        g = all_gather_rows(part, self.group)                                # [world, T, h] float32
        total = g[0].clone()
        for r in range(1, self.world):                                       # rank order: every rank adds identically
            total += g[r]
        return total.to(x.dtype)
