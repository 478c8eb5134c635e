"""The device-resident layer chain (grouped projections -> SwiGLU -> down -> RMS-norm -> ... -> lm_head/argmax)
on a small stack, against the same chain evaluated with the CPU oracle. bf16 rounding of the intermediates may
flip single elements when the two sides differ in the last fp32 bits, so the chain is compared with a tolerance
and the token only when the oracle's winning margin is clear."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_small_stack_matches_oracle_chain(runtime, oracle):
    import torch

    from qwen38_metal_b200.stack import SyntheticStack

    layers, hidden, inter, vocab = 3, 512, 1024, 1000
    rows = (96, 32, 16, 48, 1024, 1024)  # four attention-side projections, then gate and up
    stack = SyntheticStack(runtime, layers=layers, hidden=hidden, inter=inter, vocab=vocab, layer_rows=rows,
                           seed=77, misalign=2)
    stream = torch.cuda.current_stream().cuda_stream
    stack.reset_input(stream)
    torch.cuda.synchronize()
    x = oracle.bf16_to_f32(stack.x.view(torch.int16).cpu().numpy().view(np.uint16))
    assert np.array_equal(oracle.f32_to_bf16(x), oracle.synth_bf16(77, stack.x0_tensor, hidden))
    stack.decode_token(stream)
    runtime.device_status()

    tensor = 0
    for _ in range(layers):
        outs = []
        for n in rows:
            w, s, b = oracle.synth_q4(77, tensor, n, hidden)
            outs.append(oracle.matmul_factored_f32(x, w, s, b, n)[0])
            tensor += 1
        h = oracle.bf16_to_f32(oracle.f32_to_bf16(oracle.swiglu(outs[-2], outs[-1])))
        w, s, b = oracle.synth_q4(77, tensor, hidden, inter)
        tensor += 1
        d = oracle.matmul_factored_f32(h, w, s, b, hidden)[0]
        x = oracle.bf16_to_f32(oracle.f32_to_bf16(d / np.sqrt(np.mean(d.astype(np.float64) ** 2) + 1e-6).astype(np.float32)))
    got_d = stack.d.cpu().numpy()
    assert oracle.rel_l2(got_d, d) <= 2e-3
    # the last layer's side projections are computed too (they are outputs of the grouped launch)
    for i in range(len(rows) - 2):
        assert oracle.rel_l2(stack.outs[i].cpu().numpy()[:rows[i]], outs[i]) <= 2e-3
    w, s, b = oracle.synth_q4(77, tensor, vocab, hidden)
    logits = oracle.matmul_factored_f32(x, w, s, b, vocab)[0]
    order = np.sort(logits)
    if order[-1] - order[-2] > 1e-2 * abs(order[-1]):
        assert int(stack.token.item()) == int(np.argmax(logits))


@pytest.mark.parametrize("misalign", [0, 2, 6])
def test_persistent_chain_matches_launch_per_stage_path(runtime, oracle, misalign):
    """One cooperative launch for the whole token against the same stack run stage by stage."""
    import torch

    from qwen38_metal_b200.stack import SyntheticStack

    layers, hidden, inter, vocab = 3, 512, 1024, 1000
    rows = (96, 32, 16, 48, 1024, 1024)
    stack = SyntheticStack(runtime, layers=layers, hidden=hidden, inter=inter, vocab=vocab, layer_rows=rows,
                           seed=78, misalign=misalign)
    stream = torch.cuda.current_stream().cuda_stream
    stack.reset_input(stream)
    torch.cuda.synchronize()
    x0 = stack.x.clone()
    stack.decode_token(stream)
    runtime.device_status()
    ref_d, ref_token = stack.d.clone(), int(stack.token.item())
    ref_outs = [o.clone() for o in stack.outs]
    ref_x = stack.x.clone()

    chain = stack.build_chain()
    for _ in range(2):  # twice: barrier words, counters and partial slots must be reusable
        stack.x.copy_(x0)
        stack.d.zero_()
        stack.token.zero_()
        torch.cuda.synchronize()
        chain.run(stream)
        runtime.device_status()
        assert oracle.rel_l2(stack.d.cpu().numpy(), ref_d.cpu().numpy()) <= 2e-3
        for got, ref in zip(stack.outs, ref_outs):
            assert oracle.rel_l2(got.cpu().numpy(), ref.cpu().numpy()) <= 2e-3
        assert torch.equal(stack.x, ref_x) or oracle.rel_l2(stack.x.float().cpu().numpy(), ref_x.float().cpu().numpy()) <= 1e-2
        logits = stack.logits.cpu().numpy()
        assert int(stack.token.item()) == int(np.argmax(logits))
        order = np.sort(logits)
        if order[-1] - order[-2] > 1e-2 * abs(order[-1]):
            assert int(stack.token.item()) == ref_token
    chain.close()
