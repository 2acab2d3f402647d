"""Compare the plain implementation with the reference's own compiled CPU model, once.

What it does (run from the repository root; needs the reference project's sources and a
C++ compiler, no GPU):

1. builds the reference's CPU libraries and tools with CMake (tests, benchmarks and
   CUDA switched off), in a scratch folder;
2. writes the two tiny model folders with the engine's random-weights mode;
3. converts each with the reference's ``tools/convert_hf_llama.py`` and its
   ``helix_model_pack``;
4. asks the reference's ``helix_model_inspect`` for the last-position logits of several
   prefixes and for a greedy continuation;
5. writes ``tests/golden/tiny_<name>.json``: the token ids, the reference's logits
   (as float32 hex strings, exact), its greedy tokens and a checksum of the weights;
6. keeps the smaller model as the reference's packer wrote it, ``tests/golden/tiny_A.helix``
   (half a megabyte): the engine loads that file and must generate the same tokens.

``tests/test_plain_reference.py`` recomputes the same quantities with
``tests/plain_llama.py`` and compares them with the committed files, so the plain
implementation stays anchored to the reference without the reference being present.

    python tests/golden/make_golden.py --reference /path/to/helix-runtime --scratch /tmp/golden
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import plain_llama  # noqa: E402
from tiny_configs import make_folder, tiny_config  # noqa: E402

PREFIX_LENGTHS = {"A": (1, 5, 17, 31), "B": (1, 9, 40, 100)}
GREEDY = {"A": (17, 12), "B": (9, 20)}      # (prompt length, new tokens)


def run(command, **kwargs):
    completed = subprocess.run(command, capture_output=True, text=True, **kwargs)
    if completed.returncode != 0:
        raise SystemExit(f"command failed: {' '.join(map(str, command))}\n"
                         f"{completed.stdout}\n{completed.stderr}")
    return completed.stdout


def weights_checksum(folder: str) -> str:
    with open(os.path.join(folder, "model.safetensors"), "rb") as source:
        return hashlib.sha256(source.read()).hexdigest()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True)
    parser.add_argument("--scratch", required=True)
    options = parser.parse_args()
    scratch = os.path.abspath(options.scratch)
    build = os.path.join(scratch, "refbuild")
    os.makedirs(scratch, exist_ok=True)
    if not os.path.exists(os.path.join(build, "tools", "helix_model_inspect")):
        run(["cmake", "-S", options.reference, "-B", build, "-DHELIX_ENABLE_CUDA=OFF",
             "-DHELIX_BUILD_TESTS=OFF", "-DHELIX_BUILD_BENCHMARKS=OFF",
             "-DHELIX_FETCH_DEPENDENCIES=OFF", "-DCMAKE_BUILD_TYPE=Release"])
        run(["cmake", "--build", build, "-j", "8"])
    packer = os.path.join(build, "tools", "helix_model_pack")
    inspect = os.path.join(build, "tools", "helix_model_inspect")
    converter = os.path.join(options.reference, "tools", "convert_hf_llama.py")

    for name in ("A", "B"):
        config = tiny_config(name)
        folder = make_folder(scratch, name, storage_dtype="float32")
        helix_file = os.path.join(scratch, f"tiny_{name}.helix")
        run([sys.executable, converter, "--input", folder, "--output", helix_file,
             "--packer", packer, "--force", "--quiet"])
        if name == "A":
            shutil.copyfile(helix_file, os.path.join(ROOT, "tests", "golden", "tiny_A.helix"))
        rng = np.random.default_rng(100 + ord(name))
        tokens = [int(t) for t in rng.integers(0, config.vocab_size, size=max(PREFIX_LENGTHS[name]))]
        record = {"config": config.to_dict(), "weights_sha256": weights_checksum(folder),
                  "tokens": tokens, "last_logits_hex": {}, "greedy": {}}
        plain = plain_llama.PlainModel(folder)
        worst = 0.0
        for length in PREFIX_LENGTHS[name]:
            prefix = tokens[:length]
            out = run([inspect, helix_file, "--last-logits", ",".join(map(str, prefix))])
            line = [l for l in out.splitlines() if l.startswith("last_logits_hex=")][0]
            values = [float.fromhex(v) for v in line.split("=", 1)[1].split(",")]
            reference = np.asarray(values, dtype=np.float32)
            record["last_logits_hex"][str(length)] = [float(v).hex() for v in reference]
            mine = plain.logits(prefix)[-1]
            worst = max(worst, float(np.abs(mine - reference).max()))
        prompt_length, new_tokens = GREEDY[name]
        out = run([inspect, helix_file, "--greedy-tokens",
                   ",".join(map(str, tokens[:prompt_length])), str(new_tokens)])
        line = [l for l in out.splitlines() if l.startswith("generated_token_ids=")][0]
        greedy = [int(v) for v in line.split("=", 1)[1].split(",") if v]
        record["greedy"] = {"prompt_length": prompt_length, "tokens": greedy}
        mine = plain.greedy(tokens[:prompt_length], new_tokens)
        record["plain_max_abs_error_when_made"] = worst
        record["plain_greedy_equal_when_made"] = mine == greedy
        path = os.path.join(ROOT, "tests", "golden", f"tiny_{name}.json")
        with open(path, "w", encoding="utf-8") as output:
            json.dump(record, output, indent=1)
            output.write("\n")
        print(f"tiny {name}: plain vs reference max abs error {worst:.3e}; "
              f"greedy equal: {mine == greedy}; wrote {path}")


if __name__ == "__main__":
    main()
