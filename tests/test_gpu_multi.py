"""Multi-GPU tests (need >= 2 GPUs on the box; skipped otherwise): one process per GPU over NCCL.

* head sharding: each rank runs the single-GPU kernel on its heads, no data-path collective; the
  concatenation equals the single-GPU result bit for bit and matches the oracle.
* sequence parallel (Ulysses): rows start sharded, all-to-all to heads, fused call, all-to-all back; every
  rank's rows match the oracle within the parity tolerance - once with torch.distributed carrying the
  all-to-all and once through the library's own NCCL communicator (one C call per step), bit-identical.
* the host-side watchdog: krea_cuda_dist_sync with a 1 ms limit while every rank's stream is busy.
"""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    import oracle
    from krea_image_b200 import dist as kd
    from krea_image_b200 import binding, ops, synth

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        H, T, gh, gw = 4, 128, 24, 32
        S = T + gh * gw                      # 896 rows: 448 per rank
        rng = np.random.default_rng(123)     # same data on every rank
        qkv = synth.f32_to_bf16_bits(rng.standard_normal((1, S, 3 * H * 128)).astype(np.float32))
        wq = rng.uniform(0.5, 1.5, 128).astype(np.float32)
        wk = rng.uniform(0.5, 1.5, 128).astype(np.float32)
        cos, sin = synth.rope_tables_axial2d(T, gh, gw)
        want = oracle.joint_attention(qkv, 1, S, H, wq, wk, cos, sin)[0]
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        d_wq, d_wk, d_cos, d_sin = dev(wq), dev(wk), dev(cos), dev(sin)
        kc = ops.KreaCuda(rank)
        kc.set_stream(torch.cuda.current_stream())
        ld = 3 * H * 128
        x = torch.from_numpy(qkv[0].view(np.int16)).cuda().view(torch.bfloat16)

        # ---- head sharding: my heads only, straight out of the fused rows (no collective) ----
        h0, h1 = kd.head_range(H, world, rank)
        nh = h1 - h0
        o = torch.zeros((S, nh * 128), dtype=torch.bfloat16, device="cuda")
        xf = x.view(-1)
        kc.joint_attention(xf[h0 * 128:], xf[(H + h0) * 128:], xf[(2 * H + h0) * 128:], o, S, S, nh, ld, ld, ld, nh * 128,
                           d_wq, d_wk, d_cos, d_sin)
        kc.wait()
        got = o.float().cpu().numpy()
        ref = want[:, h0 * 128:h1 * 128]
        rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert rel <= 5e-3 and np.abs(got - ref).max() <= 2e-2, f"head shard rank {rank}: {rel}"
        # identical to what one GPU computes for all heads
        o_all = torch.zeros((S, H * 128), dtype=torch.bfloat16, device="cuda")
        kc.joint_attention(xf, xf[H * 128:], xf[2 * H * 128:], o_all, S, S, H, ld, ld, ld, H * 128, d_wq, d_wk, d_cos, d_sin)
        kc.wait()
        assert torch.equal(o_all[:, h0 * 128:h1 * 128].contiguous().view(torch.int16), o.view(torch.int16))

        # ---- sequence parallel ----
        plan = kd.UlyssesPlan(S, H, world)
        lo, hi = plan.row_range(rank)
        ua = kd.UlyssesAttention(kc, plan, kd.TorchGroup())
        out = ua(x[lo:hi].contiguous(), d_wq, d_wk, d_cos, d_sin)
        kc.wait()
        got = out.float().cpu().numpy()
        ref = want[lo:hi]
        rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert rel <= 5e-3 and np.abs(got - ref).max() <= 2e-2, f"ulysses rank {rank}: {rel}"
        assert torch.equal(out.view(torch.int16), o_all[lo:hi].contiguous().view(torch.int16))   # same kernels, same bits

        # ---- the same through the library's own communicator: one C call per step, first with peer
        # stores (pack kernels and the attention epilogue write into the other GPU's memory, NCCL only
        # for barriers), then with NCCL transfers ----
        xl = x[lo:hi].contiguous()
        assert kc.dist_size() == 0 and kc.dist_rank() == -1 and kc.dist_exchange_mode() == "none"
        for mode in ("p2p", "nccl"):
            os.environ["KREA_CUDA_SEQPAR_EXCHANGE"] = mode
            assert kd.init_native(kc) == (rank, world)
            assert kc.dist_size() == world and kc.dist_rank() == rank
            assert kc.dist_exchange_mode() == mode, kc.dist_exchange_mode()
            na = kd.NativeUlyssesAttention(kc, plan)
            for _ in range(3):   # later calls reuse the workspace
                out2 = na(xl, d_wq, d_wk, d_cos, d_sin)
                kc.dist_sync(60000)
                assert torch.equal(out2.view(torch.int16), out.view(torch.int16)), mode
                out2.zero_()
            if mode == "p2p":
                kc.dist_shutdown()
        # the two exchanges on their own: there and back again
        rl, cl = plan.rows_local, plan.cols_local
        q_heads = torch.zeros((S, cl), dtype=torch.bfloat16, device="cuda")
        kc.reshard_seq_to_heads(xl, q_heads, rl, cl, ld, 0)
        kc.dist_sync(60000)
        assert torch.equal(q_heads.view(torch.int16), x[:, rank * cl:(rank + 1) * cl].contiguous().view(torch.int16))
        back = torch.zeros((rl, H * 128), dtype=torch.bfloat16, device="cuda")
        kc.reshard_heads_to_seq(q_heads, back, rl, cl, H * 128, 0)
        kc.dist_sync(60000)
        assert torch.equal(back.view(torch.int16), xl[:, :H * 128].contiguous().view(torch.int16))
        kc.dist_shutdown()
        assert kc.dist_size() == 0

        # ---- the watchdog's timeout branch, on a communicator that every rank has joined: no rank is missing and
        # no collective is in flight; a few milliseconds of ordinary kernels are queued and dist_sync is given 1 ms.
        # It must report E_TIMEOUT, give the communicator up, and leave the handle serving single-GPU calls.
        assert kd.init_native(kc) == (rank, world)
        Sb, Hb = 8192, 8
        xb = torch.randn((Sb, 3 * Hb * 128), device="cuda").to(torch.bfloat16).view(-1)
        ob = torch.empty((Sb, Hb * 128), dtype=torch.bfloat16, device="cuda")
        cb, sb = (dev(t) for t in synth.rope_tables_axial2d(0, 64, 128))
        ldb = 3 * Hb * 128
        torch.cuda.synchronize()
        for _ in range(40):                      # about 0.2 ms each
            kc.joint_attention(xb, xb[Hb * 128:], xb[2 * Hb * 128:], ob, Sb, Sb, Hb, ldb, ldb, ldb, Hb * 128, d_wq, d_wk, cb, sb)
        with pytest.raises(ops.KreaCudaError) as e:
            kc.dist_sync(1)
        assert e.value.code == binding.E_TIMEOUT, str(e.value)
        assert kc.dist_size() == 0 and kc.dist_rank() == -1
        kc.wait()                                # the queued kernels finish; nothing was left waiting on a peer
        o_again = torch.zeros((S, H * 128), dtype=torch.bfloat16, device="cuda")
        kc.joint_attention(xf, xf[H * 128:], xf[2 * H * 128:], o_again, S, S, H, ld, ld, ld, H * 128, d_wq, d_wk, d_cos, d_sin)
        kc.wait()
        assert torch.equal(o_again.view(torch.int16), o_all.view(torch.int16))
        kc.dist_shutdown()
        kc.close()
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_head_sharding_and_ulysses_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
