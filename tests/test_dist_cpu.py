"""World-size-2 gloo test of the multi-GPU host logic (head ranges, the Ulysses reshard plan and its
all-to-all plumbing) on CPU tensors.  The CUDA pack / unpack kernels are replaced here by torch index
expressions that state the same formulas; the kernels themselves are checked on the GPU."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

from krea_image_b200 import dist as kd


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def pack_ref(src, dst, nranks, rows, cols, src_ld, col0):
    for p in range(nranks):
        dst[p].copy_(src[:rows, col0 + p * cols: col0 + (p + 1) * cols])


def unpack_ref(src, dst, nranks, rows, cols, dst_ld, col0):
    for p in range(nranks):
        dst[:rows, col0 + p * cols: col0 + (p + 1) * cols].copy_(src[p])


def _worker(rank, world, port, S, H):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = kd.UlyssesPlan(S, H, world)
        comm = kd.TorchGroup()
        g = torch.Generator().manual_seed(7)
        full = torch.randn(S, 3 * H * 128, generator=g).to(torch.bfloat16)      # same on every rank
        lo, hi = plan.row_range(rank)
        local = full[lo:hi].contiguous()
        alloc = lambda shape, name: torch.empty(shape, dtype=torch.bfloat16)
        h0, h1 = kd.head_range(H, world, rank)
        parts = []
        for t in range(3):
            got = kd.seq_to_heads(plan, comm, local, t * H * 128, pack_ref, alloc)
            want = full[:, t * H * 128 + h0 * 128: t * H * 128 + h1 * 128]
            assert torch.equal(got, want), f"tensor {t} rank {rank}"
            parts.append(got.clone())
        # the way back: pretend O = Q (head-sharded) and check every rank gets its rows of all heads
        back = kd.heads_to_seq(plan, comm, parts[0].contiguous(), unpack_ref, alloc)
        assert torch.equal(back, full[lo:hi, :H * 128])
    finally:
        torch.distributed.destroy_process_group()


@pytest.mark.timeout(120)
def test_ulysses_reshard_roundtrip_world2():
    port = _free_port()
    mp.spawn(_worker, args=(2, port, 12, 4), nprocs=2, join=True)


def test_head_ranges_and_plan_validation():
    assert [kd.head_range(24, 8, r) for r in (0, 7)] == [(0, 3), (21, 24)]
    assert kd.head_range(24, 1, 0) == (0, 24)
    with pytest.raises(ValueError):
        kd.head_range(24, 5, 0)
    with pytest.raises(ValueError):
        kd.UlyssesPlan(66048, 24, 7)
    p = kd.UlyssesPlan(66048, 24, 8)
    assert p.rows_local == 8256 and p.heads_local == 3 and p.cols_local == 384 and p.row_range(7) == (57792, 66048)
