"""Tiny configurations, model folders and comparison helpers shared by the tests."""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "plain"))
import qwen2_plain as plain  # noqa: E402

# Tolerances, relative to the largest reference logit of the comparison.  float32 against the
# float64 oracle (the worst seen over a thousand random configurations and the long-context decoding
# tests is 7e-6); bfloat16 (weights, activations and cache rounded to 8 bits of mantissa; the worst
# seen over the same runs is 1.6e-2, the tiny configurations stay under 7e-3).
TOL_F32 = 2e-5
TOL_BF16 = 2e-2

# Three tiny configurations that differ in every size and option: heads and groups (2 per kv head,
# MQA with 3, one per kv head), head size (16, 32, and 48 given apart from hidden/heads), width and
# vocabulary that are no powers of two, layers, eps, theta, tying, window and frequency scaling.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 128, "use_sliding_window": False,
    "hidden_act": "silu",
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "intermediate_size": 200, "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 256, "use_sliding_window": False,
}
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 112, "vocab_size": 300, "rope_theta": 500000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 512,
    "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 1,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
}
# Head size 64 with three query heads per kv head: in bfloat16 this one runs the tensor-core attention.
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 176, "vocab_size": 200, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 1024,
    "use_sliding_window": True, "sliding_window": 100, "max_window_layers": 1,
}
TINY = {"D": (TINY_D, dict(std=0.05, bias_std=0.05), 16),
        "A": (TINY_A, dict(std=0.02, bias_std=0.02), 8),
        "B": (TINY_B, dict(std=0.02, bias_std=0.05), 16),
        "C": (TINY_C, dict(std=0.05, bias_std=0.05), 16)}     # name -> (config, init, page size)


def make_model(root, name, seed=0, dtype=torch.float32, config=None, **init):
    """Write a model folder with random weights under `root` and return its path."""
    from beglin_b200.weights import write_random_model
    cfg, base_init, _ = TINY[name] if config is None else (config, {}, None)
    kw = dict(base_init)
    kw.update(init)
    folder = os.path.join(str(root), f"{name}_{seed}_{str(dtype).split('.')[-1]}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_random_model(folder, cfg, seed, dtype=dtype, **kw)
    return folder


_PLAIN_CACHE = {}


def plain_model(folder):
    if folder not in _PLAIN_CACHE:
        _PLAIN_CACHE[folder] = plain.read_folder(folder, torch.float64)
    return _PLAIN_CACHE[folder]


def plain_logits(folder, ids):
    """float64 logits [T, vocab] of the whole sequence from the plain implementation."""
    cfg, w = plain_model(folder)
    key = (folder, tuple(ids))
    if key not in _PLAIN_CACHE:
        _PLAIN_CACHE[key] = plain.forward(cfg, w, list(ids))
    return _PLAIN_CACHE[key]


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    want = want.to(torch.float64).cpu()
    got = got.to(torch.float64).cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def seeded_ids(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def follows_plain(folder, prompt, out, tol=TOL_BF16):
    """Generated tokens against the plain implementation, teacher-forced (the engine's own tokens are the
    continuation, so one near-tie does not send the rest of the comparison elsewhere): each token's plain
    logit lies within `tol` (of the row's largest magnitude) of the row's maximum, and wherever the plain top
    two are further apart than that, the token IS the plain argmax.  Returns how many tokens were pinned so."""
    logits = plain_logits(folder, list(prompt) + list(out))
    pinned = 0
    for k, tok in enumerate(out):
        row = logits[len(prompt) + k - 1]
        top = torch.topk(row, 2).values
        slack = tol * float(row.abs().max())
        assert float(top[0] - row[tok]) <= slack, (k, tok)
        if float(top[0] - top[1]) > slack:
            assert tok == int(row.argmax()), (k, tok)
            pinned += 1
    return pinned
