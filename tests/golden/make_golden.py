#!/usr/bin/env python3
"""Make the golden files of this folder with the reference's own C code.

popixoxipop-collab/beglin's model code (qwen_infer.c) needs Apple's Accelerate and ARM NEON and does
not compile on an x86 Linux host, so whole-model outputs of the reference cannot be made here.  Its
loaders and its frequency-scaling header do compile with plain gcc.  This script compiles, into a
scratch folder, hf_config.c + hf_config_verify.c, safetensors_load.c + safetensors_quants.c +
safetensors_verify.c, and a six-line driver around rope_llama3_scale.h, and runs them on model
folders written by this framework's random-weights mode:

    config_<name>.txt        the fields the reference reads from config.json (hf_config_verify.c)
    checksums_<name>.txt     one weighted checksum per tensor (safetensors_verify.c:24-27)
    rope_scale_<name>.txt    the llama3 frequency ratios (rope_llama3_scale.h:18-28)

tests/test_golden.py compares this framework's readers and the plain implementation with these files
(and, where the reference tree and gcc are present, with fresh runs of the same programs).

    python tests/golden/make_golden.py /path/to/reference
"""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

ROPE_DRIVER = r'''
#include <stdio.h>
#include <stdlib.h>
#include "rope_llama3_scale.h"
int main(int argc, char **argv) {
    float theta = atof(argv[1]); int hd = atoi(argv[2]);
    float factor = atof(argv[3]), low = atof(argv[4]), high = atof(argv[5]), orig = atof(argv[6]);
    for (int i = 0; i < hd / 2; i++) printf("%d %.9g\n", i, rope_llama3_scale(theta, hd, factor, low, high, orig, i));
    return 0;
}
'''


def build_tools(ref: str, out: str) -> dict:
    """Compile the reference's verify programs from `ref` into `out`; returns name -> executable."""
    tools = {}
    cc = ["gcc", "-O1", "-w", "-I", ref]
    subprocess.run(cc + [f"{ref}/hf_config.c", f"{ref}/hf_config_verify.c", "-o", f"{out}/hf_config_verify", "-lm"], check=True)
    tools["config"] = f"{out}/hf_config_verify"
    subprocess.run(cc + [f"{ref}/safetensors_load.c", f"{ref}/safetensors_quants.c", f"{ref}/hf_config.c",
                         f"{ref}/safetensors_verify.c", "-o", f"{out}/safetensors_verify", "-lm"], check=True)
    tools["checksums"] = f"{out}/safetensors_verify"
    with open(f"{out}/rope_driver.c", "w") as f:
        f.write(ROPE_DRIVER)
    subprocess.run(cc + [f"{out}/rope_driver.c", "-o", f"{out}/rope_driver", "-lm"], check=True)
    tools["rope"] = f"{out}/rope_driver"
    return tools


def run_tools(tools: dict, folder: str) -> dict:
    """The three outputs for one model folder."""
    out = {}
    out["config"] = subprocess.run([tools["config"], f"{folder}/config.json"], check=True, capture_output=True, text=True).stdout
    out["checksums"] = subprocess.run([tools["checksums"], f"{folder}/model.safetensors"], check=True, capture_output=True, text=True).stdout
    cfg = json.load(open(f"{folder}/config.json"))
    rs = cfg.get("rope_scaling")
    if rs:
        hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
        args = [cfg["rope_theta"], hd, rs["factor"], rs["low_freq_factor"], rs["high_freq_factor"],
                rs["original_max_position_embeddings"]]
        out["rope_scale"] = subprocess.run([tools["rope"]] + [str(a) for a in args], check=True, capture_output=True, text=True).stdout
    return out


# (name, tiny configuration, seed, stored type): the folders the golden files describe
CASES = [("A", 21, "float32"), ("B", 22, "bfloat16"), ("C", 23, "float16")]


def case_folder(root: str, name: str, seed: int, dtype: str) -> str:
    import torch
    from helpers import TINY
    from beglin_b200.weights import write_random_model
    cfg, init, _ = TINY[name]
    folder = os.path.join(root, f"golden_{name}")
    write_random_model(folder, cfg, seed, dtype=getattr(torch, dtype), **init)
    return folder


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference tree>")
    ref = sys.argv[1]
    with tempfile.TemporaryDirectory() as tmp:
        tools = build_tools(ref, tmp)
        for name, seed, dtype in CASES:
            outs = run_tools(tools, case_folder(tmp, name, seed, dtype))
            for kind, text in outs.items():
                with open(os.path.join(HERE, f"{kind}_{name}.txt"), "w") as f:
                    f.write(text)
                print(f"wrote {kind}_{name}.txt ({len(text)} bytes)")


if __name__ == "__main__":
    main()
