"""Expert parallelism over the GPUs of one box: contiguous expert ranges per rank (ds41f ref/inference/model.py:863-870),
one exchange step per layer.

Two schemes, both on `torch.distributed` process groups (NCCL over NVLink on GPUs, gloo in the CPU tests):

  reduce (decode, and prefill when every rank holds every row): every rank routes all rows (the router is replicated
      and deterministic, so all ranks choose the same experts), runs only its own experts and the f32 partial sums
      `[rows][H]` are all-reduced; the shared expert runs on rank 0 and travels in the same message
      (model.py:901-902: `dist.all_reduce(y)`).

  all-to-all (prefill / ragged batches with the rows partitioned over the ranks): a row is sent once to every rank that
      owns at least one of its picked experts, together with its picks; the owner returns the row's f32 partial sum; the
      source adds the partial sums in rank order (a fixed order, so the result is deterministic) and the shared
      expert's output, which it computes itself for its own rows.

The exchange is plumbing: what is computed between the collectives is the CUDA library (or, in the CPU tests, the
oracle passed in as `local_compute`).

On GPUs the decode scheme has a second form, `PeerReduce`: the ranks' partial sums live in symmetric (peer-mapped) memory
and one kernel of the library on every GPU adds them over NVLink and rounds (`dsgx_finalize_peers`), instead of an NCCL
all-reduce followed by the rounding kernel.
"""
import ctypes as C

import torch
import torch.distributed as dist


def expert_range(rank, world, E):
    """Rank's experts [lo, hi): contiguous ids, as the reference's MoE.__init__ partitions them."""
    assert E % world == 0, "the number of experts must be divisible by the number of ranks"
    n = E // world
    return rank * n, (rank + 1) * n


def allreduce_partials(yr, ys, group=None):
    """yr, ys: f32 [rows][H] partial sums of this rank (ys zero on ranks without the shared expert) -> summed in place."""
    buf = torch.stack([yr, ys])
    dist.all_reduce(buf, group=group)
    yr.copy_(buf[0])
    ys.copy_(buf[1])
    return yr, ys


def dispatch_plan(idx, world, E):
    """idx int32 [T][topk] -> (send_rows: list per destination of the local row numbers it gets, mask [T][world])."""
    n = E // world
    owner = torch.div(idx, n, rounding_mode="floor")                       # [T][topk] rank owning each pick
    mask = torch.zeros(idx.shape[0], world, dtype=torch.bool, device=idx.device)
    mask.scatter_(1, owner.long(), True)
    return [torch.nonzero(mask[:, d], as_tuple=False).flatten() for d in range(world)], mask


def all_to_all_experts(x, idx, w, E, local_compute, group=None):
    """x bf16 [T_local][H], idx int32 [T_local][topk], w f32 [T_local][topk]: this rank's rows.
    local_compute(x_rows, idx_rows, w_rows) -> f32 [rows][H]: the partial sum of the rows over THIS rank's experts only.
    Returns f32 [T_local][H]: the routed experts' sum of every local row (the shared expert is the caller's)."""
    world = dist.get_world_size(group)
    T, H = x.shape
    topk = idx.shape[1]
    dev = x.device
    send_rows, _ = dispatch_plan(idx, world, E)
    send_counts = torch.tensor([r.numel() for r in send_rows], dtype=torch.int64, device=dev)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    order = torch.cat(send_rows) if T else torch.zeros(0, dtype=torch.int64, device=dev)
    # three messages per direction: rows, picks, weights
    xs, ids, ws = x[order].contiguous(), idx[order].contiguous(), w[order].contiguous()
    n_in = int(sum(rc))
    xr = torch.empty(n_in, H, dtype=x.dtype, device=dev)
    ir = torch.empty(n_in, topk, dtype=idx.dtype, device=dev)
    wr = torch.empty(n_in, topk, dtype=w.dtype, device=dev)
    for out, inp in ((xr, xs), (ir, ids), (wr, ws)):
        dist.all_to_all_single(out, inp, output_split_sizes=rc, input_split_sizes=sc, group=group)
    y_in = local_compute(xr, ir, wr) if n_in else torch.zeros(0, H, dtype=torch.float32, device=dev)
    y_back = torch.empty(order.numel(), H, dtype=torch.float32, device=dev)
    dist.all_to_all_single(y_back, y_in.contiguous(), output_split_sizes=sc, input_split_sizes=rc, group=group)
    # add the partial sums in rank order
    acc = torch.zeros(T, H, dtype=torch.float32, device=dev)
    off = 0
    for d in range(world):
        rows = send_rows[d]
        if rows.numel():
            acc.index_add_(0, rows, y_back[off:off + rows.numel()])
        off += rows.numel()
    return acc


class PeerReduce:
    """The buffers of the peer-memory reduction of a decode step: this rank's partial sums and flag words in symmetric
    memory (every rank of the box maps every rank's), the device arrays of peer pointers, the step state.

        pr = PeerReduce(H, shared_rank=0)
        yr, ys = pr.parts(pr.launched + 1)                 # where this step's expert kernels write
        step.run(layer_w, x, finalize=False, yr=yr, ys=ys)
        out = pr.finalize(M)                               # the reduced, rounded rows: the same bits on every rank

    The half of the buffer a step uses follows the parity of its number (1, 2, ...): a CUDA graph that holds an even
    number of steps can be replayed any number of times."""

    FLAG_BYTES = 256

    def __init__(self, H, rows_cap=8, shared_rank=0, group=None, sliced=False):
        """sliced: the form for many rows (a prefill's pass): every rank reduces 1 / world of the rows and stores the
        rounded rows into every rank's output buffer, which then lives in the symmetric memory too."""
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        self._lib = _lib
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.H, self.rows_cap = H, rows_cap
        dev = torch.device("cuda", torch.cuda.current_device())
        half = 2 * rows_cap * H
        parts_bytes = 2 * half * 4
        out_bytes = rows_cap * H * 2 if sliced else 0
        self.buf = symm_mem.empty(self.FLAG_BYTES + parts_bytes + out_bytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group=group)
        ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.flags = torch.tensor(ptrs, dtype=torch.int64, device=dev)
        self.parts_ptrs = torch.tensor([p + self.FLAG_BYTES for p in ptrs], dtype=torch.int64, device=dev)
        self.state = torch.zeros(2, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        f = self.buf[self.FLAG_BYTES:self.FLAG_BYTES + parts_bytes].view(torch.float32).view(2, 2, rows_cap, H)
        self._parts = f
        if sliced:
            o = self.FLAG_BYTES + parts_bytes
            self.out = self.buf[o:].view(torch.bfloat16).view(rows_cap, H)
            self.outs = torch.tensor([p + o for p in ptrs], dtype=torch.int64, device=dev)
            self.done = torch.tensor([p + 128 for p in ptrs], dtype=torch.int64, device=dev)   # the flag block's second half
            outs_p, done_p = self.outs.data_ptr(), self.done.data_ptr()
        else:
            self.out = torch.zeros(rows_cap, H, dtype=torch.bfloat16, device=dev)
            outs_p, done_p = None, None
        self.sliced = sliced
        self.set = _lib.PeerSet(self.parts_ptrs.data_ptr(), self.flags.data_ptr(), self.state.data_ptr(), self.rank,
                                self.world, rows_cap, shared_rank, outs_p, done_p)
        self.launched = 0  # finalize launches executed or captured so far (the host's copy of the step counter)
        torch.cuda.synchronize()
        dist.barrier(group)  # every rank's flags are zero before anyone signals

    def parts(self, step):
        """(yr, ys) f32 [rows_cap][H] of step number `step` (1, 2, ...) in this rank's symmetric buffer."""
        return self._parts[step & 1, 0], self._parts[step & 1, 1]

    def finalize(self, M, count=True, out=None):
        """out: where the rounded rows go (default: this object's device buffer; a pinned host tensor is written in place)."""
        lib = self._lib.lib()
        assert out is None or not self.sliced, "the sliced form writes the symmetric output rows"
        dst = self.out if out is None else out
        rc = lib.dsgx_finalize_peers(C.byref(self.set), M, self.H, C.c_void_p(dst.data_ptr()),
                                     C.c_void_p(self.status.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc:
            raise self._lib.DsgxError(rc, "dsgx_finalize_peers")
        if count:
            self.launched += 1
        return dst[:M]

    def finalize_norm(self, M, norm_w, res=None, eps=1e-6, norm_mode=0, add_f32=False, count=True):
        """The reduction with the residual add and the next block's RMSNorm in the same kernel:
        returns (out, h, normed) = (bf16(v), bf16(res + out), RMSNorm(h)), each bf16 [M][H], the same bits on every rank."""
        lib = self._lib.lib()
        assert not self.sliced
        dev = self.out.device
        h, normed = (torch.empty(M, self.H, dtype=torch.bfloat16, device=dev) for _ in range(2))
        an = self._lib.AddNorm(res.data_ptr() if res is not None else None, h.data_ptr(), norm_w.data_ptr(), normed.data_ptr(),
                               eps, norm_mode, int(add_f32), 0)
        rc = lib.dsgx_finalize_peers_norm(C.byref(self.set), M, self.H, C.c_void_p(self.out.data_ptr()), C.byref(an),
                                          C.c_void_p(self.status.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc:
            raise self._lib.DsgxError(rc, "dsgx_finalize_peers_norm")
        if count:
            self.launched += 1
        return self.out[:M], h, normed
