"""Command line in the manner of the reference's ``helix_generate`` (examples/generate.cpp).

    helix_generate --model MODEL [--max-new-tokens N] [--eos TOKEN] TOKEN [TOKEN ...]

Token ids in, token ids out; there is no tokenizer.  ``--model`` is a Helix model file
(``MODEL.helix``, what the reference's command takes, examples/generate.cpp:22-27) or a model
folder with ``config.json`` and safetensors.  ``--model``, ``--max-new-tokens``
(default 32) and ``--eos`` have the reference's names and meanings, and the output has its
three lines: ``generated_token_ids``, ``stop_reason``, ``cached_token_count``.  Added here:
``--temperature`` and ``--seed`` (the reference samples greedily only), ``--dtype``,
``--page-size``, and ``--random-weights SEED``, which first writes a model folder with
seeded random weights from the ``config.json`` found in ``--model``.
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Optional, Sequence


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(
        prog="helix_generate",
        description="Generate token ids with the B200 engine (token ids in, token ids out).")
    parser.add_argument("--model", required=True,
                        help="a Helix model file (MODEL.helix) or a model folder with config.json "
                             "and model.safetensors")
    parser.add_argument("--max-new-tokens", type=int, default=32)
    parser.add_argument("--eos", type=int, default=None, help="token id that ends generation")
    parser.add_argument("--temperature", type=float, default=0.0,
                        help="0 selects greedily (the default)")
    parser.add_argument("--seed", type=int, default=0, help="seed of the sampling stream")
    parser.add_argument("--dtype", choices=("bfloat16", "float32", "bf16", "fp32"),
                        default="bfloat16")
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                        help="write model.safetensors with N(0, 0.02) weights from this seed "
                             "into --model (which must hold a config.json) before loading")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("tokens", nargs="+", type=int, metavar="TOKEN", help="prompt token ids")
    return parser


def main(arguments: Optional[Sequence[str]] = None) -> int:
    parser = build_parser()
    options = parser.parse_args(arguments)
    if options.max_new_tokens < 0:
        parser.error("--max-new-tokens must be a nonnegative integer")
    try:
        from .config.registry import load_config
        from .engine.engine import Engine, write_random_model

        if options.random_weights is not None:
            _, config = load_config(options.model)
            write_random_model(options.model, config, options.random_weights)
        engine = Engine.from_pretrained(options.model, dtype=options.dtype, device=options.device,
                                        page_size=options.page_size, max_running_requests=1)
        result = engine.generate([options.tokens], max_new_tokens=options.max_new_tokens,
                                 eos_token=options.eos, temperature=options.temperature,
                                 seed=options.seed)[0]
    except Exception as error:  # the reference prints the message and its usage, exit code 1
        print(f"helix_generate: {error}", file=sys.stderr)
        parser.print_usage(sys.stderr)
        return 1
    print("generated_token_ids:" + "".join(f" {token}" for token in result.generated_tokens))
    print(f"stop_reason: {result.stop_reason}")
    print(f"cached_token_count: {result.cached_token_count}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
