"""The plain implementation against logits the reference's own model code produced on the CPU."""
import importlib.util
from pathlib import Path

import numpy as np
import torch

from damendaemon_b200.weights import write_random_model
from plain_gpt2 import PlainGpt2

GOLDEN = Path(__file__).parent / "golden"
spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)


def test_plain_matches_reference_logits(tmp_path):
    golden = np.load(GOLDEN / "reference_logits.npz")
    for name, (config, seed, groups) in make_golden.CASES.items():
        folder = write_random_model(tmp_path / name, config, seed, "float32", name_prefix="transformer.")
        plain = PlainGpt2(folder)
        for gi, lengths in enumerate(groups):
            sequences = make_golden.prompts_for(config, lengths, seed + gi)
            want = golden[f"{name}.{gi}"]
            for r, (ids, n) in enumerate(zip(sequences, lengths)):
                logits = plain.logits(ids)
                for step in range(make_golden.DECODE_STEPS + 1):
                    got = logits[n - 1 + step].float().numpy()
                    assert np.abs(got - want[step, r]).max() < 2e-6, (name, gi, r, step)
                    assert got.argmax() == want[step, r].argmax()


def test_plain_options_change_the_result(tmp_path, tiny_configs):
    """exact-erf gelu and inverse-layer scaling are not silently ignored."""
    base = {**tiny_configs["B"], "activation_function": "gelu_new", "scale_attn_by_inverse_layer_idx": False}
    ids = list(range(3, 40))
    ref = PlainGpt2(write_random_model(tmp_path / "base", base, 1)).logits(ids)
    for change in ({"activation_function": "gelu"}, {"scale_attn_by_inverse_layer_idx": True}):
        other = PlainGpt2(write_random_model(tmp_path / str(len(change) + hash(str(change)) % 97), {**base, **change}, 1)).logits(ids)
        assert (other - ref).abs().max() > 1e-6


def test_plain_window_attention():
    from plain_gpt2 import causal_attention
    torch.manual_seed(0)
    q, k, v = (torch.randn(12, 2, 16, dtype=torch.float64) for _ in range(3))
    full = causal_attention(q, k, v, 0.25)
    win = causal_attention(q, k, v, 0.25, window=4)
    assert torch.allclose(full[:4], win[:4])
    assert not torch.allclose(full[8:], win[8:])
    # a window query sees exactly itself and the 3 keys before it
    ref = causal_attention(q[5:9], k[5:9], v[5:9], 0.25)
    assert torch.allclose(win[8], ref[3])


def test_plain_activations_against_the_library_functions():
    """The exact-erf gelu, which the reference refuses (damendaemon/config.py:301), and gelu_new, which it computes as
    F.gelu(u, approximate='tanh') (damendaemon/gpt2.py:63), held to torch's own functions in float64."""
    from plain_gpt2 import gelu_erf, gelu_new
    u = torch.cat([torch.linspace(-12, 12, 4001, dtype=torch.float64), torch.tensor([0.0, -0.0, 1e-30, -1e-30, 40.0, -40.0],
                                                                                     dtype=torch.float64)])
    assert (gelu_erf(u) - torch.nn.functional.gelu(u, approximate="none")).abs().max() < 1e-14
    assert (gelu_new(u) - torch.nn.functional.gelu(u, approximate="tanh")).abs().max() < 1e-14
    assert (gelu_erf(u) - gelu_new(u)).abs().max() > 1e-4          # the two are different functions
