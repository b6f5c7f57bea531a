"""Writes the .crseq golden fixture: a ResNet-8 (8x8 images, 10 classes) saved by the REFERENCE's own codec
(seio/modelcache/codec.cu:8-39 saveSequence, compiled from the reference tree into oracle/_ref/relink_driver by
oracle/build_relink.sh) from seeded parameters.

    python tests/golden/make_crseq_golden.py [out_dir]      (on a machine with a GPU and the relink driver built)

Outputs resnet8_hw8.crseq and resnet8_hw8_crseq.json (the flat parameter layout and seed the values came from, so a
CPU-only test can regenerate them and compare with what the file holds).
"""
import hashlib
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
sys.path.insert(0, ROOT)

BLOCKS, BATCH, HW, CLASSES, KEY = 1, 2, 8, 10, "crseq_golden"


def golden_params(entries, n_params):
    """Seeded parameters with BatchNorm's gamma / beta moved off their 1 / 0 defaults, so an exchange would show."""
    from crusaderbackend_b200 import seeds
    from crusaderbackend_b200.train import seeded_params
    host = seeded_params(entries, n_params, KEY)
    for i, e in enumerate(entries):
        if e["kind"].startswith("bn"):
            host[e["offset"]:e["offset"] + e["size"]] += 0.1 * seeds.uniform_pm1((e["size"],), KEY, "bnp", i)
    return host


def file_order(entries, host):
    """The parameter section as the reference writes it: operand order, BatchNorm beta before gamma
    (seann/operands/seblas/BatchNorm.cu:50-55)."""
    parts, i = [], 0
    while i < len(entries):
        e = entries[i]
        if e["kind"] == "bn_gamma":
            b = entries[i + 1]
            parts += [host[b["offset"]:b["offset"] + b["size"]], host[e["offset"]:e["offset"] + e["size"]]]
            i += 2
        else:
            parts.append(host[e["offset"]:e["offset"] + e["size"]])
            i += 1
    return np.concatenate(parts)


def main(out_dir):
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    driver = os.path.join(ROOT, "oracle", "_ref", "relink_driver")
    ctx = Context(0, math="fp32", sync=True)
    tr = ResNetTrainer(ctx, batch=BATCH, blocks_per_stage=BLOCKS, image_hw=HW, classes=CLASSES)
    host = golden_params(tr.entries, tr.n_params)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "resnet8_hw8.crseq")
    with tempfile.TemporaryDirectory() as tmp:
        fin = os.path.join(tmp, "in.bin")
        host.tofile(fin)
        subprocess.run([driver, "save", str(BLOCKS), str(BATCH), str(HW), str(CLASSES), fin, path], check=True,
                       env=dict(os.environ, CRUSADER_QUIET="1"))
    want = file_order(tr.entries, host)
    meta = dict(blocks=BLOCKS, batch=BATCH, hw=HW, classes=CLASSES, key=KEY, epoch=3, n_params=tr.n_params,
                entries=[dict(kind=e["kind"], offset=e["offset"], size=e["size"], dims=list(e["dims"])) for e in tr.entries],
                param_floats=int(want.size), params_sha256=hashlib.sha256(want.tobytes()).hexdigest())
    with open(os.path.join(out_dir, "resnet8_hw8_crseq.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print(path, os.path.getsize(path), "bytes")
    tr.close()
    ctx.close()


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
