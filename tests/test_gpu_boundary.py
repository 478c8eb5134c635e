"""Promises of the boundary that need a device to check: one runtime shared by several host threads
(the reference shares one MetalRuntime between generation lanes, src/api.rs:608-616, and serialises on its pool
mutex, src/metal_runtime.rs:3627-3678), a device wait that runs out and is reported as CommandFailed with the
runtime still usable afterwards (src/metal_runtime.rs:3661-3663), and the host-buffer token step."""
import threading

import numpy as np
import pytest

from helpers import upload_matrix

pytestmark = pytest.mark.gpu


def test_two_host_threads_share_one_runtime(runtime, oracle):
    """Two threads call one handle at the same time, one with decode matvecs (fp32 and bf16 activations, grouped), one
    with prompt-row matmuls; every result must equal what the same call returns single-threaded."""
    k = 1024
    mats = []
    for i, n in enumerate((96, 200, 64)):
        w, s, b = oracle.synth_q4(501, i, n, k)
        mats.append(upload_matrix(runtime, w, s, b, offset=2 if i == 1 else 0))
    x1 = oracle.bf16_to_f32(oracle.synth_bf16(501, 900, k))
    xb = oracle.synth_bf16(501, 901, k)
    xm = oracle.synth_bf16(501, 902, 24 * k)
    expect_vec = runtime.q4_affine_matvec_mapped_batch(x1, mats)
    expect_bf = runtime.q4_affine_matvec_mapped_batch(xb, mats[:2])
    expect_mm = runtime.q4_affine_matmul_mapped_batch(xm, 24, mats[1:])
    errors = []

    def decode_lane():
        try:
            for _ in range(25):
                for got, ref in zip(runtime.q4_affine_matvec_mapped_batch(x1, mats), expect_vec):
                    assert np.array_equal(got, ref)
                for got, ref in zip(runtime.q4_affine_matvec_mapped_batch(xb, mats[:2]), expect_bf):
                    assert np.array_equal(got, ref)
        except Exception as exc:  # noqa: BLE001 - reported by the main thread
            errors.append(exc)

    def prefill_lane():
        try:
            for _ in range(25):
                for got, ref in zip(runtime.q4_affine_matmul_mapped_batch(xm, 24, mats[1:]), expect_mm):
                    assert np.array_equal(got, ref)
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=decode_lane), threading.Thread(target=prefill_lane), threading.Thread(target=decode_lane)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[0]


def test_a_wait_that_runs_out_is_reported_and_the_runtime_stays_usable(runtime, oracle):
    """A two-rank chain whose second rank never launches: its barrier word lives in a second local arena that nobody
    adds to, so the first cross-GPU wait of rank 0 sees one arrival of two. With a small poll limit the kernel gives up
    within milliseconds, every block leaves, the device reports CommandFailed, the chain refuses to run again, and an
    ordinary chain on the same runtime still matches the per-stage path. Nothing faults or hangs: the wait returns
    by itself."""
    import torch

    from qwen38_metal_b200.runtime import Q4RuntimeError
    from qwen38_metal_b200.stack import SyntheticStack

    kw = dict(layers=2, hidden=512, inter=1024, vocab=1000, layer_rows=(96, 32, 1024, 1024), seed=81, misalign=2)
    stream = torch.cuda.current_stream().cuda_stream
    half = SyntheticStack(runtime, rank=0, world=2, **kw)
    half.reset_input(stream)
    mine, _ = runtime.arena_create(half.sharded_arena_bytes())
    nobody, _ = runtime.arena_create(half.sharded_arena_bytes())
    chain = half.build_chain_sharded(None, arenas=[mine, nobody])
    chain.set_spin_limit(2000)
    chain.run(stream)
    with pytest.raises(Q4RuntimeError) as err:
        runtime.device_status()
    assert err.value.kind == "CommandFailed"
    with pytest.raises(Q4RuntimeError) as err:
        chain.run(stream)
    assert err.value.kind == "ActivationPoolPoisoned"
    chain.close()
    runtime.device_status()  # the flag was consumed: the device is healthy

    whole = SyntheticStack(runtime, **kw)
    whole.reset_input(stream)
    torch.cuda.synchronize()
    x0 = whole.x.clone()
    whole.decode_token(stream)
    runtime.device_status()
    ref_d, ref_token = whole.d.clone(), int(whole.token.item())
    good = whole.build_chain()
    whole.x.copy_(x0)
    good.run(stream)
    runtime.device_status()
    assert oracle.rel_l2(whole.d.cpu().numpy(), ref_d.cpu().numpy()) <= 2e-3
    assert int(whole.token.item()) == int(np.argmax(whole.logits.cpu().numpy()))
    order = np.sort(whole.logits.cpu().numpy())
    if order[-1] - order[-2] > 1e-2 * abs(order[-1]):
        assert int(whole.token.item()) == ref_token
    good.close()


def test_host_buffer_token_step(runtime, oracle):
    """q4b_chain_run: host slice in, token out, equal to the device-resident run of the same chain."""
    import torch

    from qwen38_metal_b200.stack import SyntheticStack

    stack = SyntheticStack(runtime, layers=2, hidden=512, inter=1024, vocab=1000, layer_rows=(96, 1024, 1024), seed=82, misalign=2)
    stream = torch.cuda.current_stream().cuda_stream
    stack.reset_input(stream)
    torch.cuda.synchronize()
    x_bits = stack.x.view(torch.int16).cpu().numpy().view(np.uint16).copy()
    chain = stack.build_chain()
    chain.run(stream)
    runtime.device_status()
    token, best = int(stack.token.item()), float(stack.best.item())
    stack.x.zero_()
    stack.token.zero_()
    torch.cuda.synchronize()
    got_token, got_best = chain.run_host(x_bits)
    assert (got_token, got_best) == (token, best)
    chain.close()
