"""The worker's command line, in the reference's manner.

Reference (src/worker/main.cpp:35-88): ``pih-worker --lock LOCK_PATH [--serve
LOOPBACK_PORT | --generate-tokens ID,ID,... --max-tokens COUNT]``; the token
mode prints one line ``{"schema":"pih.token-generation-result.v1",
"token_ids":[...],"finish_reason":"stop|length","prompt_tokens":n,
"completion_tokens":m}`` (src/worker/worker_bootstrap.cpp:584-591), runs with
``top_p = 1`` and ``seed = 7`` (:551-552), takes at most 65 536 prompt ids and
``1 <= COUNT <= 65536`` (main.cpp:47-65), refuses a trailing comma, and
reports failures as ``pih_worker_failed: <reason>`` with exit code 1; a wrong
command line prints the usage and exits with 2.

Here the model folder stands where the lock file stood (there are no
plugins to lock), ``--serve`` does not exist (servers are out of scope), and
the sampling options that the reference fixes in code can be given;
``--logprobs`` and ``--top-logprobs N`` add what its sampler returns with
every token (plugins/model-qwen3/qwen3_sampler.cpp:132-149) to the line.
"""
from __future__ import annotations

import json
import sys

USAGE = ("usage: pih-worker --model MODEL_DIR --generate-tokens ID,ID,... --max-tokens COUNT "
         "[--dtype bfloat16|float32] [--temperature T] [--top-p P] [--top-k K] [--seed S] "
         "[--ignore-eos] [--logprobs] [--top-logprobs N] [--page-size N] [--max-cache-tokens N]\n"
         "       pih-worker --random-model MODEL_DIR --config CONFIG_JSON --seed S [--sigma X] "
         "[--store bfloat16|float32]\n")


def _parse_tokens(text: str):
    if not text or len(text) > 512 * 1024:
        raise ValueError("prompt_tokens_invalid")
    if text.endswith(","):
        raise ValueError("prompt_tokens_trailing_comma")
    out = []
    for part in text.split(","):
        if not part.isdigit() or len(out) >= 65536:
            raise ValueError("prompt_tokens_invalid")
        out.append(int(part))
    return out


def _options(argv):
    opts, flags = {}, {"--ignore-eos", "--logprobs"}
    i = 0
    while i < len(argv):
        a = argv[i]
        if a in flags:
            opts[a] = True
            i += 1
        elif a.startswith("--") and i + 1 < len(argv):
            opts[a] = argv[i + 1]
            i += 2
        else:
            return None
    return opts


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    opts = _options(argv)
    known = {"--model", "--generate-tokens", "--max-tokens", "--dtype", "--temperature", "--top-p", "--top-k",
             "--seed", "--ignore-eos", "--logprobs", "--top-logprobs", "--page-size", "--max-cache-tokens", "--random-model", "--config",
             "--sigma", "--store"}
    if opts is None or set(opts) - known:
        sys.stderr.write(USAGE)
        return 2
    try:
        if "--random-model" in opts:
            if "--config" not in opts or "--seed" not in opts:
                sys.stderr.write(USAGE)
                return 2
            import torch
            from ..config.registry import config_from_dict
            from ..weights import write_random_model
            with open(opts["--config"], "r", encoding="utf-8") as f:
                config = config_from_dict(json.load(f))
            store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[opts.get("--store", "bfloat16")]
            write_random_model(opts["--random-model"], config, seed=int(opts["--seed"]),
                               sigma=float(opts.get("--sigma", 0.02)), dtype=store)
            print(json.dumps({"schema": "pih.random-model.v1", "model": opts["--random-model"],
                              "seed": int(opts["--seed"])}))
            return 0
        if not {"--model", "--generate-tokens", "--max-tokens"} <= set(opts):
            sys.stderr.write(USAGE)
            return 2
        tokens = _parse_tokens(opts["--generate-tokens"])
        if not opts["--max-tokens"].isdigit() or not 1 <= int(opts["--max-tokens"]) <= 65536:
            raise ValueError("maximum_tokens_invalid")
        maximum = int(opts["--max-tokens"])
        from ..cache import DEFAULT_PAGE_SIZE
        from ..engine import Engine
        params = {"temperature": float(opts.get("--temperature", 0.0)), "top_p": float(opts.get("--top-p", 1.0)),
                  "seed": int(opts.get("--seed", 7)), "ignore_eos": bool(opts.get("--ignore-eos", False))}
        if "--top-k" in opts:
            params["top_k"] = int(opts["--top-k"])
        if "--logprobs" in opts or "--top-logprobs" in opts:       # the result then carries "logprobs" (and "top_logprobs")
            params["logprobs"] = True
            params["top_logprobs"] = int(opts.get("--top-logprobs", 0))
        engine = Engine(opts["--model"], opts.get("--dtype", "bfloat16"),
                        page_size=int(opts.get("--page-size", DEFAULT_PAGE_SIZE)),
                        max_cache_tokens=int(opts["--max-cache-tokens"]) if "--max-cache-tokens" in opts
                        else len(tokens) + maximum + 64,
                        maximum_batch_sequences=1)
        result = engine.complete(tokens, max_tokens=maximum, **params)
        engine.rt.ops.check_errors()
        print(json.dumps(result, separators=(",", ":")))
        return 0
    except Exception as error:  # the reference reports every failure this way (main.cpp:78-84)
        sys.stderr.write(f"pih_worker_failed: {error}\n")
        return 1


if __name__ == "__main__":
    raise SystemExit(main())
