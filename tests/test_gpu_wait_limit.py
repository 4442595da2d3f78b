"""The attention kernel's bounded waits, exercised on purpose: a launch whose producer never requests its last K
tile (a host-set test hook) makes the wait for that tile run out after a limit of a few milliseconds.  Nothing
faults and nothing spins for longer than the limit: every CTA records where it gave up, runs to its normal exit
(tensor memory released, copies in flight awaited) and krea_cuda_sync reports KREA_CUDA_E_DEVICE with the wait
site; the status word is cleared and the next call on the same handle is bit-identical to a clean run."""
import numpy as np
import pytest
import torch

from krea_image_b200 import binding, ops, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("persist", ["0", "2"])     # the one-item kernel and the persistent one (forced on this small case)
def test_a_wait_that_runs_out_is_reported_and_the_handle_recovers(monkeypatch, persist):
    monkeypatch.setenv("KREA_CUDA_PERSIST", persist)
    kc = ops.KreaCuda(0)
    kc.set_stream(torch.cuda.current_stream())
    try:
        H, T, gh, gw = 2, 128, 16, 24
        S = T + gh * gw                                   # 512 rows: two query blocks x two heads, four key tiles each
        rng = np.random.default_rng(77)
        qkv = synth.f32_to_bf16_bits(rng.standard_normal((1, S, 3 * H * 128)).astype(np.float32))
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        wq, wk = dev(rng.uniform(0.5, 1.5, 128).astype(np.float32)), dev(rng.uniform(0.5, 1.5, 128).astype(np.float32))
        cos, sin = (dev(t) for t in synth.rope_tables_axial2d(T, gh, gw))
        x = torch.from_numpy(qkv.view(np.int16)).cuda().view(torch.bfloat16).view(-1)
        ld = 3 * H * 128

        def run():
            o = torch.zeros((S, H * 128), dtype=torch.bfloat16, device="cuda")
            kc.joint_attention(x, x[H * 128:], x[2 * H * 128:], o, S, S, H, ld, ld, ld, H * 128, wq, wk, cos, sin)
            return o

        clean = run()
        kc.wait()
        with pytest.raises(ops.KreaCudaError):
            kc.set_wait_limit(1e-7)                       # limits below a millisecond are refused
        kc.set_wait_limit(0.005)
        kc.test_drop_one_load(True)
        run()
        with pytest.raises(ops.KreaCudaError) as e:
            kc.wait()
        assert e.value.code == binding.E_DEVICE, str(e.value)
        # whichever role's wait ran out first reports its site: the tensor-core warp waiting for the K tile (2), or a
        # softmax warpgroup waiting for the scores (4) / the product (6) that never came
        assert any(f"site {n}," in str(e.value) for n in (2, 4, 5, 6)), str(e.value)
        kc.test_drop_one_load(False)
        kc.set_wait_limit(2.0)
        kc.wait()                                         # the status word was cleared: no stale error
        again = run()
        kc.wait()
        assert torch.equal(again.view(torch.int16), clean.view(torch.int16))
    finally:
        kc.close()
