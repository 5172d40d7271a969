"""Command line in the manner of the reference's `examples/local_model.rs`: the model comes from a
configuration file (here JSON with `LocalModelConfig`'s field names), the request from the flags.

    python -m cuca_b200 --config engine.json --prompt "1 15 27 4" --max-tokens 32 --temperature 0
    python -m cuca_b200 --model-dir DIR --prompt-len 128
    python -m cuca_b200 --random-weights 5 --model-config config.json --dtype bfloat16

Flags of the reference: --config, --prompt (token ids; text when the model folder brings a tokenizer.json and
the prompt is not a list of numbers), --max-tokens (default 1024), --temperature (0 is greedy; default: the
model's own). `--thinking` is accepted and ignored: chat templates are outside this engine. Ours: --model-dir,
--model-config, --random-weights SEED, --dtype, --top-k, --top-p, --seed, --prompt-len, --stop (a stop string,
may be given several times; needs the tokenizer).
It prints `load:`, `loaded on`, the generated ids (the text, with a tokenizer), and the reference's `timing:` line
on standard error.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m cuca_b200", description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", help="JSON file holding the LocalModelConfig")
    ap.add_argument("--prompt", help="token ids separated by spaces or commas; text if the folder has a tokenizer")
    ap.add_argument("--stop", action="append", default=[], help="stop string (needs the folder's tokenizer)")
    ap.add_argument("--prompt-len", type=int, help="use this many seeded random token ids as the prompt")
    ap.add_argument("--thinking", default=None, help="accepted for parity with the reference; ignored")
    ap.add_argument("--max-tokens", type=int, default=1024)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--model-dir", help="model folder (config.json + safetensors); overrides the config's source")
    ap.add_argument("--model-config", help="a config.json to run with random weights")
    ap.add_argument("--random-weights", type=int, metavar="SEED", help="draw the weights from this seed")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default=None)
    args = ap.parse_args(argv)

    from .config.engine_config import LocalModelConfig, RandomWeights
    from .engine.engine import LocalModel

    config = LocalModelConfig.from_file(args.config) if args.config else LocalModelConfig()
    if args.model_dir:
        config.source, config.model_config = args.model_dir, None
    if args.model_config:
        config.model_config, config.source = json.loads(open(args.model_config).read()), None
        config.random_weights = RandomWeights(seed=args.random_weights or 0)
    elif args.random_weights is not None and config.model_config is not None:
        config.random_weights = RandomWeights(seed=args.random_weights)
    if args.dtype:
        config.dtype = args.dtype

    started = time.perf_counter()
    model = LocalModel.load(config)
    print(f"load: {time.perf_counter() - started:.1f} s", file=sys.stderr)
    import torch
    print(f"loaded on {torch.cuda.get_device_name(model.core.rt.device)} ({config.dtype}, "
          f"{model.kv_cache_bytes() / 2**20:.0f} MiB of K/V pages)", file=sys.stderr)

    vocab = model.core.spec.vocab_size
    as_text = False
    if args.prompt:
        words = args.prompt.replace(",", " ").split()
        if model.text is not None and not all(w.lstrip("-").isdigit() for w in words):
            prompt, as_text = model.tokenize(args.prompt), True
        else:
            prompt = [int(t) for t in words]
    else:
        import numpy as np
        prompt = np.random.default_rng(1).integers(0, vocab, size=args.prompt_len or 16).tolist()

    asked = time.perf_counter()
    first = [None]

    def on_token(seq, tok):
        if first[0] is None:
            first[0] = time.perf_counter() - asked
        if not as_text:
            print(tok, end=" ", flush=True)

    def on_text(seq, fragment):
        if as_text:
            print(fragment, end="", flush=True)

    gen = model.generate(prompt, max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k,
                         top_p=args.top_p, seed=args.seed, on_token=on_token, stop=args.stop, on_text=on_text)
    print()
    usage = gen.report.usage
    if first[0] is not None:
        rest = max(time.perf_counter() - asked - first[0], 1e-9)
        print(f"timing: {usage.prompt_tokens} prompt tokens, first token after {first[0]:.2f} s "
              f"(~{usage.prompt_tokens / max(first[0], 1e-9):.2f} prompt tokens/s); {usage.completion_tokens} "
              f"completion tokens, then {max(usage.completion_tokens - 1, 0) / rest:.3f} tokens/s after the first; "
              f"finish_reason {gen.report.finish_reason}", file=sys.stderr)
    if gen.report.error:
        print(f"error: {gen.report.error}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
