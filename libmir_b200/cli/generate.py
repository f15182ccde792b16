"""Generate tokens from a model folder, in the manner of libmir's examples/generate.rs:13-71.

    bin/generate MODEL_DIR [--prompt-ids 1,2,3] [--max-tokens 256] [--temperature 0] ...

The model folder comes from the first argument or from $MODEL, as there.  libmir's example renders a
chat prompt and prints text; tokenizers and chat templates are not part of this engine, so the prompt is
given as token ids and token ids are printed (streamed as they are produced), followed by
`finish_reason=...` on a line of its own.  Options carry the names of libmir's GenerationOverrides
(models/src/generation/mod.rs:38-47) and GenerationRequest.seed; the cache options carry the names of
its CacheConfig (runtime/src/kv/cache/types.rs:57-66).
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="generate", description=__doc__.split("\n\n")[0])
    parser.add_argument("model", nargs="?", default=os.environ.get("MODEL"),
                        help="folder with config.json and *.safetensors (or $MODEL)")
    parser.add_argument("--prompt-ids", default="1", help="comma-separated token ids of the prompt; several prompts "
                        "separated by ';' run as one batch")
    parser.add_argument("--max-tokens", type=int, default=256)
    parser.add_argument("--min-tokens", type=int, default=None)
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--repetition-penalty", type=float, default=1.0)
    parser.add_argument("--seed", type=int, default=None, help="seed of the sampler (default: libmir's)")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--block-size", type=int, default=16, help="tokens in one cache page")
    parser.add_argument("--block-count", type=int, default=4096, help="cache pages")
    parser.add_argument("--prefix-cache", action="store_true",
                        help="remember full cache pages by their tokens and share them between requests that start alike")
    parser.add_argument("--max-batch-tokens", type=int, default=8192)
    parser.add_argument("--random-weights", metavar="CONFIG_JSON", default=None,
                        help="build the model this config.json describes with seeded random weights instead of "
                             "loading a folder")
    parser.add_argument("--weights-seed", type=int, default=0)
    parser.add_argument("--write-random-model", metavar="DIR", default=None,
                        help="with --random-weights: write config.json and model.safetensors to DIR and exit")
    parser.add_argument("--json", action="store_true", help="print one JSON object per request instead of a stream")
    args = parser.parse_args(argv)

    from ..config import CacheConfig, GenerationOverrides, RuntimeConfig, SchedulerConfig
    from ..engine.api import GenerationRequest, Library

    if args.write_random_model:
        if not args.random_weights:
            parser.error("--write-random-model needs --random-weights CONFIG_JSON")
        from ..weights import write_model_folder
        config = json.load(open(args.random_weights))
        folder = write_model_folder(args.write_random_model, config, seed=args.weights_seed, dtype=args.dtype)
        print(f"wrote {folder}/config.json and {folder}/model.safetensors")
        return 0
    if not args.model and not args.random_weights:
        parser.error("MODEL or the first argument is required")

    runtime = RuntimeConfig(kv_cache=CacheConfig(block_size=args.block_size, block_count=args.block_count,
                                                 prefix_cache=args.prefix_cache),
                            scheduler=SchedulerConfig(max_batch_tokens=args.max_batch_tokens), dtype=args.dtype)
    library = Library(runtime)
    if args.random_weights:
        model = library.load_random(json.load(open(args.random_weights)), seed=args.weights_seed)
    else:
        model = library.load(args.model)
    options = GenerationOverrides(max_tokens=args.max_tokens, min_tokens=args.min_tokens,
                                  ignore_eos=args.ignore_eos or None, temperature=args.temperature,
                                  top_p=args.top_p, top_k=args.top_k, repetition_penalty=args.repetition_penalty)
    prompts = [[int(t) for t in part.replace(" ", "").split(",") if t] for part in args.prompt_ids.split(";")]
    requests = [GenerationRequest(prompt, options, seed=args.seed, request_id=index)
                for index, prompt in enumerate(prompts)]

    if args.json or len(requests) > 1:
        for output in model.generate_batch(requests):
            print(json.dumps({"request": output.request_id, "token_ids": output.token_ids,
                              "finish_reason": output.finish_reason, "metrics": output.metrics}))
        return 0

    def on_token(token: int) -> None:
        sys.stdout.write(f"{token} ")
        sys.stdout.flush()

    output = model.generate(requests[0], on_token)
    sys.stdout.write(f"\nfinish_reason={output.finish_reason}\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
