import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


# the two tiny configurations differ in every size and option
TINY_A = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 64, "n_head": 4, "n_inner": None, "vocab_size": 512, "n_positions": 128,
    "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
    "scale_attn_by_inverse_layer_idx": False,
}
TINY_B = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 3, "n_embd": 96, "n_head": 2, "n_inner": 320, "vocab_size": 1000, "n_positions": 256,
    "layer_norm_epsilon": 1e-6, "activation_function": "gelu",
    "scale_attn_by_inverse_layer_idx": True,
}
# a third one with head size 64, the size the tensor-core attention kernels take
TINY_C = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 192, "n_head": 3, "n_inner": 400, "vocab_size": 331, "n_positions": 320,
    "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
    "scale_attn_by_inverse_layer_idx": False,
}
# and an awkward one: one layer, five heads of 16, an inner width (100) and a vocabulary (97) that are no multiple of 8
TINY_D = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 1, "n_embd": 80, "n_head": 5, "n_inner": 100, "vocab_size": 97, "n_positions": 96,
    "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
    "scale_attn_by_inverse_layer_idx": True,
}


# head size 128: in bfloat16 the mma.sync prompt kernel and the row decode kernel at the engine's level
TINY_E = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 256, "n_head": 2, "n_inner": 384, "vocab_size": 411, "n_positions": 192,
    "layer_norm_epsilon": 1e-5, "activation_function": "gelu",
    "scale_attn_by_inverse_layer_idx": False,
}
# head size 80 (a step of 16 that no tensor-core attention kernel takes): the general kernel in both dtypes; seven heads
TINY_F = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 1, "n_embd": 560, "n_head": 7, "n_inner": 600, "vocab_size": 257, "n_positions": 80,
    "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
    "scale_attn_by_inverse_layer_idx": True,
}


@pytest.fixture(scope="session")
def tiny_configs():
    return {"A": dict(TINY_A), "B": dict(TINY_B)}
