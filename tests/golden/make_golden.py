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

CASES = {
    "A": (dict(TINY_A), 0, [[5, 17], [33]]),
    "Bprime": ({**TINY_B, "activation_function": "gelu_new", "scale_attn_by_inverse_layer_idx": False}, 1, [[9, 64], [200]]),
}
DECODE_STEPS = 4


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
        write_random_model(folder, {**config, "eos_token_id": 0}, seed, "float32", name_prefix="transformer.")
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
