"""Makes tests/golden/qwen3_oracle_outputs.json: a tiny Qwen3-shaped model run through the reference
project's own CPU oracles.

The reference (GuiminChen/pih) has no whole-model forward on the CPU and no Python binding, but its per-op
oracles compile here with g++ (no CUDA needed): plugins/model-qwen3/qwen3_cpu_oracle.cpp,
qwen3_gqa_oracle.cpp, qwen3_sampler.cpp and src/core/status.cpp.  ``oracle_driver.cpp`` (ours) strings them
together in the order of the reference's execution schedule and supplies the matrix products, which the
reference leaves to cuBLASLt.  This script compiles the driver against a checkout of the reference (given
with --reference or in PIH_REFERENCE; the tree is only read), feeds it a seeded random model, and stores the
inputs' seed and the outputs as JSON.  ``tests/test_golden.py`` compares the plain implementation with these numbers; it needs
neither the reference nor a compiler.

    python tests/golden/make_golden.py --reference /path/to/pih
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from golden_model import CONFIG, TOKENS, make_weights, tensor_order  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("PIH_REFERENCE"), required="PIH_REFERENCE" not in os.environ,
                    help="a checkout of GuiminChen/pih")
    args = ap.parse_args()
    ref = args.reference
    sources = [os.path.join(ref, p) for p in ("plugins/model-qwen3/qwen3_cpu_oracle.cpp",
                                              "plugins/model-qwen3/qwen3_gqa_oracle.cpp",
                                              "plugins/model-qwen3/qwen3_sampler.cpp", "src/core/status.cpp")]
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "oracle_driver")
        cmd = ["g++", "-std=c++20", "-O1", "-I", os.path.join(ref, "include"), os.path.join(HERE, "oracle_driver.cpp"),
               *sources, "-o", exe]
        subprocess.run(cmd, check=True)
        w = make_weights()
        c = CONFIG
        lines = [f"{c['num_hidden_layers']} {c['hidden_size']} {c['intermediate_size']} {c['vocab_size']} "
                 f"{len(TOKENS)} {c['rms_norm_eps']!r}", " ".join(str(t) for t in TOKENS)]
        for name in tensor_order():
            lines.append(" ".join(repr(float(x)) for x in w[name].float().reshape(-1).tolist()))
        out = subprocess.run([exe], input="\n".join(lines) + "\n", capture_output=True, text=True, check=True).stdout
    result = {"logits": [], "attention": [], "samples": [], "philox": []}
    mode = None
    for line in out.splitlines():
        if line == "logits" or line == "samples":
            mode = line
        elif line.startswith("attention "):
            mode = "attention"
            result["attention"].append([])
        elif line.startswith("philox "):
            result["philox"].append(int(line.split()[1]))
        elif mode == "logits":
            result["logits"].append(float(line))
        elif mode == "attention":
            result["attention"][-1].append(float(line))
        elif mode == "samples":
            tok, logprob, word = line.split()
            result["samples"].append([int(tok), float(logprob), int(word)])
    result["source"] = ("GuiminChen/pih CPU oracles: plugins/model-qwen3/qwen3_cpu_oracle.cpp, qwen3_gqa_oracle.cpp, "
                        "qwen3_sampler.cpp; driver tests/golden/oracle_driver.cpp; model tests/golden_model.py")
    with open(os.path.join(HERE, "qwen3_oracle_outputs.json"), "w") as f:
        json.dump(result, f)
    print(f"wrote {len(result['logits'])} logits, {len(result['attention'])} attention outputs, "
          f"{len(result['samples'])} samples")


if __name__ == "__main__":
    main()
