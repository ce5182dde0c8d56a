"""Writes the golden vectors under tests/golden/.

Run where the reference checkout is mounted:

    python tests/golden/make_fixtures.py <path of the reference checkout>

It copies, key by key, the numbers of the reference's own MLX fixtures that pin
this path (src/cpu/testdata/attention.json read by src/cpu/attention.rs:188-221,
src/cpu/testdata/ops.json read by src/cpu/ops.rs:81-110), drops the keys of
other layers, and records the known-answer inputs of src/kv_quant.rs:319-332.
The tests read only the files written here.
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

OPS_KEYS = ["x", "w", "rms_norm", "softmax", "rope_in", "rope_positions", "rope_out"]


def main(ref):
    data = os.path.join(ref, "src", "cpu", "testdata")
    with open(os.path.join(data, "attention.json")) as f:
        att = json.load(f)
    with open(os.path.join(data, "ops.json")) as f:
        ops = json.load(f)
    with open(os.path.join(HERE, "attention_mlx.json"), "w") as f:
        json.dump(att, f, separators=(",", ":"))
    with open(os.path.join(HERE, "ops_mlx.json"), "w") as f:
        json.dump({k: ops[k] for k in OPS_KEYS}, f, separators=(",", ":"))
    # src/kv_quant.rs:319-332: a group of zeros with ones at 1 and 63.
    known = {
        "ones_at": [1, 63],
        "bits8": {"words": 16, "word0": 255 << 8, "word15": 255 << 24},
        "bits4": {"words": 8, "word0": 15 << 4, "word7": 15 << 28},
    }
    with open(os.path.join(HERE, "kv_quant_known.json"), "w") as f:
        json.dump(known, f)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_fixtures.py <path of the reference checkout>")
    main(sys.argv[1])
