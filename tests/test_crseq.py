"""The reference's .crseq model files (seio/modelcache/codec.cu:8-97).

CPU: the host-only readers against the committed fixture tests/golden/resnet8_hw8.crseq, which the reference's own
saveSequence wrote (tests/golden/make_crseq_golden.py): operand count, epoch, and the parameter section equal to the
seeded values the fixture was written from, bit for bit; malformed files are refused.
GPU: a file written by the reference's codec loads into the training executor bit-exactly, the executor's own file
for the same parameters is byte-identical to the reference's, and a file of another network is refused.
"""
import ctypes as C
import hashlib
import json
import os
import struct

import numpy as np
import pytest

from tests.golden.make_crseq_golden import file_order, golden_params

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
GOLDEN = os.path.join(ROOT, "tests", "golden", "resnet8_hw8.crseq")
META = os.path.join(ROOT, "tests", "golden", "resnet8_hw8_crseq.json")


def _inspect(lib, path):
    n, ep, pf = C.c_uint(0), C.c_uint(0), C.c_ulonglong(0)
    err = C.create_string_buffer(256)
    rc = lib.cb_crseq_inspect(str(path).encode(), C.byref(n), C.byref(ep), C.byref(pf), err, 256)
    return rc, n.value, ep.value, pf.value, err.value.decode()


def test_reader_on_the_reference_written_fixture():
    from crusaderbackend_b200 import _lib
    lib = _lib.load()
    meta = json.load(open(META))
    rc, n_ops, epoch, n_floats, msg = _inspect(lib, GOLDEN)
    assert rc == 0, msg
    # 3 stem operands, 8 per block, 3 head operands, and the two projection convolutions inside their endpoints
    assert n_ops == 3 + 8 * 3 * meta["blocks"] + 3 + 2
    assert epoch == meta["epoch"] == 3
    assert n_floats == meta["param_floats"]
    got = np.empty(n_floats, dtype=np.float32)
    err = C.create_string_buffer(256)
    assert lib.cb_crseq_read_params(GOLDEN.encode(), got.ctypes.data, n_floats, err, 256) == 0, err.value.decode()
    assert hashlib.sha256(got.tobytes()).hexdigest() == meta["params_sha256"]
    # regenerated from the seed: what the reference's codec was given, in the order it stores it
    want = file_order(meta["entries"], golden_params(meta["entries"], meta["n_params"]))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the parameter section is the tail of the file
    raw = open(GOLDEN, "rb").read()
    assert raw[-4 * n_floats:] == got.tobytes()
    assert struct.unpack("<3I", raw[:12]) == (0x7921AEDF, 3 + 8 * 3 * meta["blocks"] + 3, 3)
    # a wrong count is refused
    assert lib.cb_crseq_read_params(GOLDEN.encode(), got.ctypes.data, n_floats - 1, err, 256) != 0


def test_reader_refuses_malformed_files(tmp_path):
    from crusaderbackend_b200 import _lib
    lib = _lib.load()
    raw = open(GOLDEN, "rb").read()
    bad_magic = tmp_path / "magic.crseq"
    bad_magic.write_bytes(b"\0\0\0\0" + raw[4:])
    rc, *_, msg = _inspect(lib, bad_magic)
    assert rc != 0 and "magic" in msg
    cut = tmp_path / "cut.crseq"
    cut.write_bytes(raw[:40])
    rc, *_, msg = _inspect(lib, cut)
    assert rc != 0 and "ends inside" in msg
    unknown = tmp_path / "unknown.crseq"
    unknown.write_bytes(raw[:12] + struct.pack("<I", 0xE001) + raw[16:])   # a DenseBlock prefab id
    rc, *_, msg = _inspect(lib, unknown)
    assert rc != 0 and "operand id" in msg
    rc, *_, msg = _inspect(lib, tmp_path / "absent.crseq")
    assert rc != 0 and "cannot open" in msg


@pytest.mark.gpu
def test_reference_written_file_loads_and_executor_writes_the_same_bytes(tmp_path):
    import torch
    from crusaderbackend_b200.api import Context, CrusaderError
    from crusaderbackend_b200.train import ResNetTrainer
    from tests.test_relink_gpu import run_driver
    blocks, batch, hw, classes = 2, 4, 16, 10
    ctx = Context(0, math="fp32", sync=True)
    tr = ResNetTrainer(ctx, batch=batch, blocks_per_stage=blocks, image_hw=hw, classes=classes)
    host = golden_params(tr.entries, tr.n_params)
    fin, ref_file, own_file = tmp_path / "in.bin", tmp_path / "ref.crseq", tmp_path / "own.crseq"
    host.tofile(fin)
    run_driver("save", blocks, batch, hw, classes, fin, ref_file)   # the reference's saveSequence
    # load: every parameter tensor equals what the reference saved, bit for bit
    tr.set_params(np.zeros_like(host))
    assert tr.load_crseq(ref_file) == 3
    got = tr.params.cpu().numpy()
    for e in tr.entries:
        sl = slice(e["offset"], e["offset"] + e["size"])
        assert np.array_equal(got[sl].view(np.uint32), host[sl].view(np.uint32)), (e["kind"], e["dims"])
    # save: the same bytes as the reference's writer
    tr.save_crseq(own_file, epoch=3)
    assert own_file.read_bytes() == ref_file.read_bytes()
    # the committed fixture is a file of the same writer: load it into the matching network
    small = ResNetTrainer(ctx, batch=2, blocks_per_stage=1, image_hw=8, classes=10)
    meta = json.load(open(META))
    assert small.load_crseq(GOLDEN) == 3
    want = golden_params(meta["entries"], meta["n_params"])
    assert np.array_equal(small.params.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # and a forward/backward step on the loaded weights runs (packed filters were re-made by the load)
    x = torch.randn(2, 3, 8, 8, device="cuda")
    lab = torch.zeros(2, 10, device="cuda")
    lab[:, 1] = 1
    small.forward(x, lab)
    small.backward()
    assert np.isfinite(small.loss())
    # another network's file is refused, and the bound parameters stay as they were
    before = tr.params.clone()
    with pytest.raises(CrusaderError, match="another network"):
        tr.load_crseq(GOLDEN)
    assert torch.equal(before, tr.params)
    small.close()
    tr.close()
    ctx.close()
