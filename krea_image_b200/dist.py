"""Multi-GPU execution of the joint attention: one process per GPU, torch.distributed for the plumbing.

Attention is independent per head (the reference dispatches one threadgroup column per head,
engine/src/metal.mm:199-201), so:

  * head sharding needs no data-path collective: rank r runs the single-GPU kernel on its heads;
  * the long-sequence configuration starts sequence-sharded and is resharded Ulysses-style: an
    all-to-all turns [S/P rows, all heads] into [S rows, H/P heads] for Q, K and V, the local kernel
    runs on full sequences, and a second all-to-all brings the output rows home.  RoPE positions depend
    only on the global row index, so the prologue runs after the reshard with the global tables.

The reference is single-device; nothing here has a counterpart in it.
"""
from dataclasses import dataclass

HEAD_DIM = 128


def head_range(heads: int, nranks: int, rank: int):
    """Heads [lo, hi) owned by `rank`."""
    if heads % nranks:
        raise ValueError(f"{heads} heads do not split evenly over {nranks} ranks")
    per = heads // nranks
    return rank * per, (rank + 1) * per


@dataclass(frozen=True)
class UlyssesPlan:
    """Index arithmetic of the sequence <-> head reshard."""
    seq: int
    heads: int
    nranks: int

    def __post_init__(self):
        if self.seq % self.nranks or self.heads % self.nranks:
            raise ValueError("sequence length and head count must be multiples of the number of ranks")

    @property
    def rows_local(self) -> int:
        return self.seq // self.nranks

    @property
    def heads_local(self) -> int:
        return self.heads // self.nranks

    @property
    def cols_local(self) -> int:
        return self.heads_local * HEAD_DIM

    def row_range(self, rank: int):
        return rank * self.rows_local, (rank + 1) * self.rows_local


class TorchGroup:
    """all_to_all over a torch.distributed process group (NCCL on GPUs, gloo in CPU tests)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    def all_to_all(self, out, inp):
        if self.dist.get_backend(self.group) == "gloo":
            # gloo has no all_to_all_single for every dtype: exchange equal chunks pairwise
            outs = list(out.view(self.size, -1).unbind(0))
            ins = list(inp.view(self.size, -1).unbind(0))
            reqs = []
            for p in range(self.size):
                if p == self.rank:
                    outs[p].copy_(ins[p])
                else:
                    reqs.append(self.dist.isend(ins[p].contiguous(), p, group=self.group))
                    reqs.append(self.dist.irecv(outs[p], p, group=self.group))
            for r in reqs:
                r.wait()
        else:
            self.dist.all_to_all_single(out, inp, group=self.group)


def seq_to_heads(plan: UlyssesPlan, comm, x_local, col0: int, pack, alloc):
    """One of Q / K / V: x_local [rows_local, ld] holds all heads at columns [col0, col0 + heads*128).
    Returns [seq, cols_local]: every row of the sequence, this rank's heads.
    pack(src, dst, nranks, rows, cols_per_rank, src_ld, src_col0) fills dst [P][rows][cols_per_rank];
    alloc(shape, name) returns a (reusable) buffer: distinct names never alias."""
    P, rl, cl = plan.nranks, plan.rows_local, plan.cols_local
    send = alloc((P, rl, cl), "send")
    pack(x_local, send, P, rl, cl, x_local.shape[-1], col0)
    recv = alloc((P, rl, cl), "recv")
    comm.all_to_all(recv, send)
    return recv.view(plan.seq, cl)   # block p holds rows [p*rl, (p+1)*rl): already in sequence order


def heads_to_seq(plan: UlyssesPlan, comm, o_heads, unpack, alloc):
    """o_heads [seq, cols_local] -> [rows_local, heads*128] (this rank's rows, all heads).
    unpack(src, dst, nranks, rows, cols_per_rank, dst_ld, dst_col0) merges src [P][rows][cols] into columns."""
    P, rl, cl = plan.nranks, plan.rows_local, plan.cols_local
    recv = alloc((P, rl, cl), "recv")
    comm.all_to_all(recv, o_heads.view(P, rl, cl))   # row block p goes to rank p as it is
    out = alloc((rl, plan.heads * HEAD_DIM), "out")
    unpack(recv, out, P, rl, cl, plan.heads * HEAD_DIM, 0)
    return out


class UlyssesAttention:
    """Sequence-parallel joint attention on one rank (fused q|k|v rows in, output rows out)."""

    def __init__(self, kc, plan: UlyssesPlan, comm):
        import torch
        self.torch = torch
        self.kc, self.plan, self.comm = kc, plan, comm
        self._bufs = {}

    def _alloc(self, tag):
        torch = self.torch

        def alloc(shape, name):
            key = (tag, name, tuple(shape))
            if key not in self._bufs:
                self._bufs[key] = torch.empty(shape, dtype=torch.bfloat16, device=f"cuda:{self.kc.device}")
            return self._bufs[key]
        return alloc

    def __call__(self, qkv_local, wq, wk, cos, sin, eps=1e-6, rope_mode=0):
        """qkv_local: bf16 [rows_local, 3*heads*128] on this rank's GPU; cos/sin: f32 [seq, 64] global tables.
        Returns bf16 [rows_local, heads*128]."""
        torch, plan, kc = self.torch, self.plan, self.kc
        H = plan.heads
        kc.set_stream(torch.cuda.current_stream())
        parts = [seq_to_heads(plan, self.comm, qkv_local, t * H * HEAD_DIM, kc.reshard_pack, self._alloc(f"x{t}"))
                 for t in range(3)]
        q, k, v = parts
        o = self._alloc("o")((plan.seq, plan.cols_local), "heads")
        cl = plan.cols_local
        kc.joint_attention(q, k, v, o, plan.seq, plan.seq, plan.heads_local, cl, cl, cl, cl, wq, wk, cos, sin, eps,
                           1, rope_mode)
        return heads_to_seq(plan, self.comm, o, kc.reshard_unpack, self._alloc("r"))


def init_native(kc, group=None):
    """Creates the library's own NCCL communicator over the ranks of a torch.distributed group: rank 0
    makes the id, the process group carries its 128 bytes to the others.  Returns (rank, nranks)."""
    import torch
    import torch.distributed as dist
    rank, size = dist.get_rank(group), dist.get_world_size(group)
    box = [kc.dist_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    torch.cuda.set_device(kc.device)
    kc.dist_init(rank, size, box[0])
    return rank, size


class NativeUlyssesAttention:
    """The sequence-parallel joint attention as ONE library call per step (krea_cuda_seqpar_joint_attention):
    pack kernels, ncclSend/ncclRecv exchanges, the K normalisation pass overlapped with the exchange of V
    and Q, the attention kernel and the exchange of the output all run inside libkrea_cuda."""

    def __init__(self, kc, plan: UlyssesPlan):
        if kc.dist_size() != plan.nranks:
            raise ValueError(f"the handle's communicator has {kc.dist_size()} ranks, the plan {plan.nranks}")
        self.kc, self.plan = kc, plan
        self._out = None

    def __call__(self, qkv_local, wq, wk, cos, sin, eps=1e-6, rope_mode=0, out=None):
        """qkv_local: bf16 [rows_local, 3*heads*128]; returns bf16 [rows_local, heads*128]."""
        import torch
        plan, kc = self.plan, self.kc
        H, ld = plan.heads, qkv_local.shape[-1]
        if out is None:
            if self._out is None:
                self._out = torch.empty((plan.rows_local, H * HEAD_DIM), dtype=torch.bfloat16, device=qkv_local.device)
            out = self._out
        kc.set_stream(torch.cuda.current_stream())
        flat = qkv_local.view(-1)
        kc.seqpar_joint_attention(flat, flat[H * HEAD_DIM:], flat[2 * H * HEAD_DIM:], out, plan.seq, H, ld, ld, ld,
                                  H * HEAD_DIM, wq, wk, cos, sin, eps, 1, rope_mode)
        return out
