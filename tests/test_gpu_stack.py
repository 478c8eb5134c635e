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


def test_full_width_chain_every_stage_against_the_oracle(runtime, oracle):
    """The benchmark's kernel at the benchmark's width: hidden 5120, intermediate 17408, vocabulary 248320, two layers
    (1.1 GB of weights generated in HBM, every other projection 2 bytes off a 16-byte boundary), every stage writing
    to buffers of its own. Each stage is checked against the oracle on the inputs the GPU itself produced: sampled
    weight rows (first, middle and last 16, regenerated on the CPU) of all nine K=5120 projections, of the K=17408
    down projection and of the 248320-row lm_head at the streaming kernel's bar (relative L2 <= 1e-5); the fused
    SwiGLU vector and the RMS-normed activation element by element against the oracle's formulas (bf16 values may
    differ in the last place where the two sides' fp32 inputs to the rounding differ); the token against the argmax
    of the GPU's own logits. A second launch must reproduce every buffer bit for bit."""
    import torch

    from qwen38_metal_b200 import capi
    from qwen38_metal_b200.stack import HIDDEN, INTER, LAYER_ROWS, VOCAB, SyntheticStack

    layers, seed = 2, 4242
    stack = SyntheticStack(runtime, layers=layers, seed=seed, misalign=2)
    dev, f32, bf16 = stack.device, torch.float32, torch.bfloat16
    stream = torch.cuda.current_stream().cuda_stream
    stack.reset_input(stream)
    outs = [[torch.zeros(n, dtype=f32, device=dev) for n in LAYER_ROWS] for _ in range(layers)]
    hs = [torch.zeros(INTER, dtype=bf16, device=dev) for _ in range(layers)]
    ds = [torch.zeros(HIDDEN, dtype=f32, device=dev) for _ in range(layers)]
    xs = [stack.x] + [torch.zeros(HIDDEN, dtype=bf16, device=dev) for _ in range(layers)]  # xs[l]: input of layer l; xs[layers]: lm_head's
    logits = torch.zeros(VOCAB, dtype=f32, device=dev)
    gi, ui = len(LAYER_ROWS) - 2, len(LAYER_ROWS) - 1
    stages = []
    for l in range(layers):
        head = {"x_kind": capi.X_BF16, "src0": xs[0].data_ptr()} if l == 0 else \
               {"x_kind": capi.X_RMS, "src0": ds[l - 1].data_ptr(), "x_bf16_out": xs[l].data_ptr()}
        stages.append({**head, "k": HIDDEN, "eps": 1e-6, "jobs": [p.job for p in stack.proj[l]],
                       "outputs": [o.data_ptr() for o in outs[l]]})
        stages.append({"x_kind": capi.X_SWIGLU, "k": INTER, "src0": outs[l][gi].data_ptr(), "src1": outs[l][ui].data_ptr(),
                       "x_bf16_out": hs[l].data_ptr(), "jobs": [stack.down[l].job], "outputs": [ds[l].data_ptr()]})
    stages.append({"x_kind": capi.X_RMS, "k": HIDDEN, "eps": 1e-6, "src0": ds[-1].data_ptr(), "x_bf16_out": xs[layers].data_ptr(),
                   "jobs": [stack.lm_head.job], "outputs": [logits.data_ptr()]})
    chain = runtime.chain_create(stages, logits.data_ptr(), VOCAB, 0, stack.token.data_ptr(), stack.best.data_ptr())
    chain.run(stream)
    runtime.device_status()

    def bits(t):
        return t.view(torch.int16).cpu().numpy().view(np.uint16)

    everything = [o for layer in outs for o in layer] + ds + [logits]
    first = [t.cpu().numpy().copy() for t in everything] + [bits(t).copy() for t in hs + xs[1:]]
    token = int(stack.token.item())
    chain.run(stream)
    runtime.device_status()
    second = [t.cpu().numpy() for t in everything] + [bits(t) for t in hs + xs[1:]]
    for a, b in zip(first, second):
        assert np.array_equal(a, b)
    assert int(stack.token.item()) == token

    def sampled(tensor, n, k, x_f32, got, bar=1e-5):
        for r0 in sorted({0, (n // 2) & ~15, max(n - 16, 0)}):
            rows = min(16, n - r0)
            w, s, b = oracle.synth_q4(seed, tensor, rows, k, row0=r0)
            ref = oracle.matmul_factored_f32(x_f32, w, s, b, rows)[0]
            assert oracle.rel_l2(got[r0:r0 + rows], ref) <= bar, (tensor, r0)

    def close_bf16(got_bits, ref_f32, what):
        """bf16 vectors equal up to last-place flips on a small share of the elements."""
        ref_bits = oracle.f32_to_bf16(ref_f32)
        differ = np.count_nonzero(got_bits != ref_bits)
        assert differ <= 0.005 * got_bits.size, (what, differ)
        assert oracle.rel_l2(oracle.bf16_to_f32(got_bits), oracle.bf16_to_f32(ref_bits)) <= 2e-3, what

    tensor = 0
    for l in range(layers):
        x_in = oracle.bf16_to_f32(bits(xs[l]))
        for i, n in enumerate(LAYER_ROWS):
            sampled(tensor, n, HIDDEN, x_in, outs[l][i].cpu().numpy())
            tensor += 1
        gate, up = outs[l][gi].cpu().numpy(), outs[l][ui].cpu().numpy()
        close_bf16(bits(hs[l]), oracle.swiglu(gate, up), f"swiglu of layer {l}")
        sampled(tensor, HIDDEN, INTER, oracle.bf16_to_f32(bits(hs[l])), ds[l].cpu().numpy())
        tensor += 1
        d = ds[l].cpu().numpy()
        normed = (d / np.sqrt(np.mean(d.astype(np.float64) ** 2) + 1e-6)).astype(np.float32)
        close_bf16(bits(xs[l + 1]), normed, f"rms-norm after layer {l}")
    got_logits = logits.cpu().numpy()
    sampled(tensor, VOCAB, HIDDEN, oracle.bf16_to_f32(bits(xs[layers])), got_logits)
    assert token == int(np.argmax(got_logits))  # numpy's argmax also takes the lowest index among equals
    assert float(stack.best.item()) == float(got_logits[token])
    chain.close()


@pytest.mark.parametrize("defer", ["0", "1"])
def test_mid_width_chain_with_and_without_deferred_projections(oracle, defer, monkeypatch):
    """A stack wide enough that tiles are cut into many parts (K-major phases hold slices of the activation that do not
    start at chunk 0), run with the default plan and with projections deferred behind the barriers (two activation
    buffers, Q4B_CHAIN_DEFER=1 is latched when the runtime is created): both must match the per-stage path."""
    import torch

    from qwen38_metal_b200.runtime import CudaRuntime
    from qwen38_metal_b200.stack import SyntheticStack

    monkeypatch.setenv("Q4B_CHAIN_DEFER", defer)
    rt = CudaRuntime(0)
    try:
        stack = SyntheticStack(rt, layers=3, hidden=2048, inter=4096, vocab=3000, layer_rows=(512, 256, 128, 48, 4096, 4096),
                               seed=83, misalign=2)
        stream = torch.cuda.current_stream().cuda_stream
        stack.reset_input(stream)
        torch.cuda.synchronize()
        x0 = stack.x.clone()
        stack.decode_token(stream)
        rt.device_status()
        ref_d, ref_outs, ref_token = stack.d.clone(), [o.clone() for o in stack.outs], int(stack.token.item())
        chain = stack.build_chain()
        for _ in range(2):
            stack.x.copy_(x0)
            stack.d.zero_()
            for o in stack.outs:
                o.zero_()
            torch.cuda.synchronize()
            chain.run(stream)
            rt.device_status()
            assert oracle.rel_l2(stack.d.cpu().numpy(), ref_d.cpu().numpy()) <= 2e-3
            for got, ref in zip(stack.outs, ref_outs):
                assert oracle.rel_l2(got.cpu().numpy(), ref.cpu().numpy()) <= 2e-3
            logits = stack.logits.cpu().numpy()
            assert int(stack.token.item()) == int(np.argmax(logits))
            order = np.sort(logits)
            if order[-1] - order[-2] > 1e-2 * abs(order[-1]):
                assert int(stack.token.item()) == ref_token
        chain.close()
    finally:
        rt.close()


def test_chain_with_a_hidden_width_above_8192(runtime, oracle):
    """A hidden width of 9216: the RMS-norm rebuild holds more than two blocks of 8 inputs per thread, so the chain runs
    on the kernel instance with the long rebuild. One layer, compared stage by stage with the per-stage path."""
    import torch

    from qwen38_metal_b200.stack import SyntheticStack

    layers, hidden, inter, vocab = 1, 9216, 1024, 1000
    rows = (96, 32, 16, 48, 1024, 1024)
    stack = SyntheticStack(runtime, layers=layers, hidden=hidden, inter=inter, vocab=vocab, layer_rows=rows,
                           seed=81, misalign=2)
    stream = torch.cuda.current_stream().cuda_stream
    stack.reset_input(stream)
    torch.cuda.synchronize()
    x0 = stack.x.clone()
    stack.decode_token(stream)
    runtime.device_status()
    ref_d, ref_outs, ref_x = stack.d.clone(), [o.clone() for o in stack.outs], stack.x.clone()
    ref_token = int(stack.token.item())
    chain = stack.build_chain()
    for _ in range(2):
        stack.x.copy_(x0)
        stack.d.zero_()
        torch.cuda.synchronize()
        chain.run(stream)
        runtime.device_status()
        assert oracle.rel_l2(stack.d.cpu().numpy(), ref_d.cpu().numpy()) <= 1e-5
        for got, ref in zip(stack.outs, ref_outs):
            assert oracle.rel_l2(got.cpu().numpy(), ref.cpu().numpy()) <= 1e-5
        assert oracle.rel_l2(stack.x.float().cpu().numpy(), ref_x.float().cpu().numpy()) <= 1e-2
        logits = stack.logits.cpu().numpy()
        assert int(stack.token.item()) == int(np.argmax(logits))
        order = np.sort(logits)
        if order[-1] - order[-2] > 1e-2 * abs(order[-1]):
            assert int(stack.token.item()) == ref_token
    chain.close()
