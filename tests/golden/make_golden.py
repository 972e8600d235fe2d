"""Run the reference's own GPT-2 model code once, on the CPU, and keep its logits.

    python tests/golden/make_golden.py /path/to/reference/checkout

It writes tiny random GPT-2 folders (the seeds below), loads each through the
reference's ``ModelWeights`` and ``Gpt2Executor`` with the device patched to 'cpu'
(the reference's own test idiom, tests/test_starcoder_cpu_reference.py:27-29), and
stores last-position prefill logits and teacher-forced decode logits in
``reference_logits.npz`` beside this file. ``tests/test_plain_against_golden.py``
rebuilds the same folders and holds the plain implementation to these numbers, so
the checkout is not needed when the tests run.

Configuration A runs as it is. Configuration B uses exact-erf gelu and scaling by
inverse layer index, both of which the reference refuses (damendaemon/config.py:301-303);
"B-prime" keeps B's sizes with gelu_new and no layer scaling so that head size 48,
explicit n_inner, eps 1e-6 and 3 layers are still anchored.

Scaling by inverse layer index is anchored all the same, through an identity: dividing
the scores of layer i by (i + 1) is dividing its queries by (i + 1), and the queries
are c_attn's first third. "Bscaled" therefore gives the reference B-prime's weights
with the query columns and query bias of layer i divided by (i + 1) and the option
off, which it accepts; the test holds the plain implementation, run on the unchanged
B-prime weights WITH the option on, to those logits.
"""
import json
import sys
import tempfile
from pathlib import Path
from unittest.mock import patch

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

from conftest import TINY_A, TINY_B  # noqa: E402
from damendaemon_b200.weights import write_random_model  # noqa: E402

B_PRIME = {**TINY_B, "activation_function": "gelu_new", "scale_attn_by_inverse_layer_idx": False}
# name: (the configuration the plain implementation runs, seed, groups of prompt lengths)
CASES = {
    "A": (dict(TINY_A), 0, [[5, 17], [33]]),
    "Bprime": (dict(B_PRIME), 1, [[9, 64], [200]]),
    "Bscaled": ({**B_PRIME, "scale_attn_by_inverse_layer_idx": True}, 1, [[9, 64], [200]]),
}
DECODE_STEPS = 4


def folder_for_the_reference(folder, config, seed):
    """The model folder the reference is given for a case. A configuration with scaling by inverse layer index
    becomes one without it whose queries are divided by (layer index + 1) in the weights."""
    from damendaemon_b200.registry import architecture_of
    from damendaemon_b200.weights import write_safetensors
    if not config.get("scale_attn_by_inverse_layer_idx"):
        return write_random_model(folder, {**config, "eos_token_id": 0}, seed, "float32", name_prefix="transformer.")
    plain_config = {**config, "scale_attn_by_inverse_layer_idx": False, "eos_token_id": 0}
    arch = architecture_of(config)
    tensors = arch.random_tensors(arch.parse_config(config), seed, torch.float32)
    h = config["n_embd"]
    for i in range(config["n_layer"]):
        tensors[f"h.{i}.attn.c_attn.weight"][:, :h] /= (i + 1)        # Conv1D [in, out]: the first third of the outputs
        tensors[f"h.{i}.attn.c_attn.bias"][:h] /= (i + 1)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(arch.parse_config(plain_config).to_dict()))
    write_safetensors(folder / "model.safetensors", {"transformer." + k: v for k, v in tensors.items()})
    return folder


def prompts_for(config, lengths, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return [torch.randint(0, config["vocab_size"], (n + DECODE_STEPS,), generator=g).tolist() for n in lengths]


def main(reference_root):
    sys.path.insert(0, reference_root)
    from damendaemon.qwen2 import ModelWeights
    from damendaemon.runtime import make_executor
    out = {}
    for name, (config, seed, groups) in CASES.items():
        folder = Path(tempfile.mkdtemp())
        folder_for_the_reference(folder, config, seed)
        (folder / "tokenizer.json").write_text(json.dumps({
            "version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
            "pre_tokenizer": {"type": "Whitespace"}, "post_processor": None, "decoder": None,
            "model": {"type": "WordLevel", "vocab": {"a": 0, "b": 1}, "unk_token": "a"}}))
        (folder / "tokenizer_config.json").write_text("{}")
        with patch("damendaemon.qwen2.selected_device", return_value="cpu"), \
                patch("damendaemon.qwen2.empty_cache"), \
                patch("damendaemon.qwen2.available_memory", return_value=2 ** 34), \
                patch("damendaemon.runtime.selected_device", return_value="cpu"):
            weights = ModelWeights(str(folder), config["n_positions"])
            executor = make_executor(weights, use_graph=False, max_batch=4, kernels="torch")
        for gi, lengths in enumerate(groups):
            sequences = prompts_for(config, lengths, seed + gi)
            slots = list(range(len(lengths)))
            last = executor.prefill_batch([s[:n] for s, n in zip(sequences, lengths)], slots)
            rows = [last.float().numpy()]
            for step in range(DECODE_STEPS):
                logits, _ = executor.decode_batch([s[n + step] for s, n in zip(sequences, lengths)], slots)
                rows.append(logits.float().numpy())
            # [1 + DECODE_STEPS, requests, vocab]: logits after n, n+1, ... tokens of each sequence
            out[f"{name}.{gi}"] = np.stack(rows).astype(np.float32)
    np.savez_compressed(HERE / "reference_logits.npz", **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
