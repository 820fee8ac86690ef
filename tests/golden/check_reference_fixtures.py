"""Checks the plain implementation (tests/plain/qwen3_plain.py) against the reference
project's checked-in fixtures and writes the record ``reference_fixtures.json`` beside
this file.

The reference's model code is Pascal (no compiler for it here), so it cannot be run; what
can be read are its fixtures under ``tests/data/infer-ref/`` of the reference project:
tiny Qwen3 models (config.json, BF16 model.safetensors) with the states, logits and greedy
tokens that Hugging Face transformers computed for them in float32 (``manifest.json`` +
``tensors.bin``). This script runs the plain implementation on those models and records the
largest differences. The fixtures themselves are not copied.

    python tests/golden/check_reference_fixtures.py <reference project>/tests/data/infer-ref
"""
import hashlib
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from tests.plain import qwen3_plain as plain  # noqa: E402

SETS = ["tiny-qwen3", "tiny-qwen3/untied", "tiny-qwen3-sliding"]


def read_set(folder):
    with open(os.path.join(folder, "manifest.json")) as f:
        manifest = json.load(f)
    with open(os.path.join(folder, manifest["blob"]["file"]), "rb") as f:
        blob = f.read()
    assert hashlib.sha256(blob).hexdigest() == manifest["blob"]["sha256"]
    out = {}
    for t in manifest["tensors"]:
        dt = {"f32": np.float32, "i32": np.int32, "u8": np.uint8}[t["dtype"]]
        out[t["name"]] = np.frombuffer(
            blob[t["offset"]:t["offset"] + t["bytes"]], dtype=dt).reshape(t["shape"])
    return manifest, out


def main(root):
    record = {"source": "tests/data/infer-ref of the reference project", "sets": {}}
    for name in SETS:
        folder = os.path.join(root, name)
        config, weights = plain.read_model_folder(folder)
        manifest, ref = read_set(folder)
        cases = sorted({k.split(".")[0] for k in ref})
        entry = {"config": {k: config[k] for k in (
            "num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
            "head_dim", "intermediate_size", "vocab_size")}, "cases": {}}
        for case in cases:
            ids = ref[case + ".ids"].tolist()
            states = {}
            logits = plain.forward(config, weights, ids, states)
            states["logits"] = logits
            diffs = {}
            for key, value in ref.items():
                c, what = key.split(".", 1)
                if c == case and what in states:
                    diffs[what] = float(np.abs(states[what] - value).max())
            rec = {"tokens": len(ids), "max_abs_diff": diffs,
                   "argmax_equal": bool((logits.argmax(-1) == ref[case + ".logits"].argmax(-1)).all())}
            if case + ".greedy" in ref:
                want = ref[case + ".greedy"].tolist()
                got = plain.greedy(config, weights, ids, len(want), stop=[config.get("eos_token_id", -1)])
                rec["greedy_equal"] = got == want
                rec["greedy"] = got
            entry["cases"][case] = rec
        record["sets"][name] = entry
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.json")
    with open(out, "w") as f:
        json.dump(record, f, indent=1, sort_keys=True)
    print(json.dumps(record, indent=1, sort_keys=True))


if __name__ == "__main__":
    main(sys.argv[1])
