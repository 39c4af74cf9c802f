"""Llama-3.1-8B layer sizes (hidden 4096, 32 heads / 8 kv heads of 128, intermediate 14336, vocabulary
128256, llama3 rope scaling), two layers so that the plain implementation can follow on the CPU.
Checks the kernels at the sizes the benchmark runs: 32-bit against the plain implementation under
different cuts, bfloat16 within its tolerance."""
import numpy as np
import pytest
import torch

import plain_llama
from gpu_common import BF16_REL_LARGE, need_gpu, note_worst
from replay_util import InProcessReplayer, gather, peak_tokens, trace_mixed, trace_portions, trace_whole

pytestmark = pytest.mark.gpu

LARGE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 4096,
    "intermediate_size": 14336, "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8,
    "max_position_embeddings": 131072, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}


@pytest.fixture(scope="module")
def large_folder(tmp_path_factory):
    from torchinferno_b200.weights.random_init import write_random_model
    folder = tmp_path_factory.mktemp("large")
    write_random_model(LARGE, folder, seed=5)
    return folder


@pytest.fixture(scope="module")
def large_reference(large_folder):
    g = torch.Generator().manual_seed(77)
    requests = {f"r{i}": torch.randint(0, LARGE["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate([70, 33, 130])}
    config, weights = plain_llama.read_model_folder(large_folder, dtype=torch.float32)
    want = {k: plain_llama.forward(config, weights, v).double().numpy() for k, v in requests.items()}
    return requests, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_large_layer_sizes_under_every_cut(large_folder, large_reference, dtype):
    need_gpu()
    requests, want = large_reference
    for maker in (trace_whole, trace_portions, trace_mixed):
        steps, index = maker(requests)
        replayer = InProcessReplayer(large_folder, dtype, max_tokens=peak_tokens(steps))
        rows = gather(replayer.run(steps), index)
        worst = 0.0
        for (name, pos), got_list in rows.items():
            ref = want[name]
            for got in got_list:
                assert np.isfinite(got).all()
                err = np.abs(got.astype(np.float64) - ref[pos]).max()
                # the plain implementation runs in float32 here (the model is too large for float64 on the
                # CPU), so its own rounding counts: 1e-4 of the largest logit in 32-bit
                bound = (1e-4 if dtype == "float32" else BF16_REL_LARGE) * np.abs(ref).max()
                worst = max(worst, err / bound)
                assert err <= bound, f"{maker.__name__} {name}@{pos} ({dtype}): {err:.3e} > {bound:.3e}"
        note_worst(f"8B layer sizes, short prompts, {maker.__name__} [{dtype}]", worst)
        del replayer
        torch.cuda.empty_cache()


def test_long_decoding_at_these_sizes_is_the_same_with_and_without_dependent_launch(large_folder):
    """At the 8B layer sizes kernels really overlap when they are launched as dependents (the decode attention
    fetches old keys while the rotary kernel runs, the output projection its weights while the attention drains).
    300 decoded tokens for 1 and for 8 requests at contexts of 600 to 1,200 tokens must come out the same with
    that switched off, and the same when run again."""
    need_gpu()
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import load_model, make_runner
    from torchinferno_b200.kernels import ops
    model = load_model(large_folder, dtype="bfloat16")
    histories = {}
    try:
        with torch.inference_mode():
            for on in (True, False, True):
                ops.set_dependent_launch(on)
                for batch in (1, 8):
                    runner = make_runner(model, page_size=16, max_tokens=batch * 1300, max_requests=batch)
                    g = torch.Generator().manual_seed(batch)
                    firsts = []
                    for i in range(batch):
                        prompt = torch.randint(0, LARGE["vocab_size"], (600 + 37 * i,), generator=g).tolist()
                        firsts.append(int(runner.step([StepEntry(i, prompt, [len(prompt) - 1])]).argmax()))
                    history = runner.decode_loop(list(range(batch)), firsts, 300).cpu()
                    runner.raise_on_device_error()
                    if (batch, on) in histories:
                        assert torch.equal(histories[(batch, on)], history)
                    histories[(batch, on)] = history
    finally:
        ops.set_dependent_launch(True)
    for batch in (1, 8):
        assert torch.equal(histories[(batch, True)], histories[(batch, False)])
