"""CPU-only: the deploy-artifact loader (host C++ in engine_io.cu) against artifacts
written by inference.save_deploy, the reference's validation rules
(src/inference_serialization.cpp:919-1033) and, where built, the reference's own loader."""
import json
import zipfile

import numpy as np
import pytest

import oracle
from munet_b200 import MuNetError
from munet_b200.inference import inspect_artifact, save_deploy

CFG = {"type": "Sequential", "layers": [
    {"type": "Linear", "in_features": 3, "out_features": 2, "bias": True}, {"type": "ReLU"}]}
TENSORS = {"0.weight": np.arange(6, dtype=np.float32).reshape(3, 2), "0.bias": np.zeros(2, np.float32)}


def rewrite(src, dst, drop=(), replace=None, compress=False):
    """Copy an artifact member by member, dropping / replacing some."""
    replace = replace or {}
    with zipfile.ZipFile(src) as zin, zipfile.ZipFile(
            dst, "w", zipfile.ZIP_DEFLATED if compress else zipfile.ZIP_STORED) as zout:
        for name in zin.namelist():
            key = name[:-4]
            if key in drop:
                continue
            if key in replace:
                import io
                buf = io.BytesIO()
                np.save(buf, replace[key])
                zout.writestr(name, buf.getvalue())
            else:
                zout.writestr(name, zin.read(name))


def test_round_trip(tmp_path):
    p = str(tmp_path / "m.npz")
    save_deploy(p, CFG, TENSORS)
    info = inspect_artifact(p)
    assert info["config"] == CFG
    assert info["tensors"] == {"0.bias": {"dtype": 0, "shape": [2]}, "0.weight": {"dtype": 0, "shape": [3, 2]}}
    if oracle.have_ref():  # the reference's own loader accepts what save_deploy writes
        ok, msg = oracle.ref().load_npz_ok(p)
        assert ok, msg


def test_dtypes_and_producers(tmp_path):
    p = str(tmp_path / "m.npz")
    save_deploy(p, {"type": "Embedding", "num_embeddings": 4, "embedding_dim": 2},
                {"weight": np.ones((4, 2), np.float16)}, producer="munet_nn")
    assert inspect_artifact(p)["tensors"]["weight"] == {"dtype": 1, "shape": [4, 2]}
    with pytest.raises(ValueError):
        save_deploy(p, CFG, {"0.weight": np.zeros((3, 2), np.float64)})


@pytest.mark.parametrize("mutation,message", [
    (dict(replace={"__format_name__": np.array("other")}), "Unsupported serialization format name"),
    (dict(replace={"__format_revision__": np.array(2, dtype=np.int64)}), "format revision"),
    (dict(replace={"__producer__": np.array("someone")}), "Unsupported serialization producer"),
    (dict(replace={"__artifact_kind__": np.array("checkpoint")}), "artifact kind"),
    (dict(replace={"__default_load_mode__": np.array("train")}), "deploy load mode"),
    (dict(replace={"__contains_training_state__": np.array(True)}), "training-only state"),
    (dict(replace={"__tensor_names__": np.array(json.dumps(["0.weight"]))}), "manifest does not match"),
    (dict(drop=("__config__",)), "does not contain architecture config"),
    (dict(replace={"0.weight": np.zeros((3, 2), np.float64)}), "Unsupported npy dtype"),
    (dict(compress=True), "Compressed npz entries are not supported"),
])
def test_rejections_follow_the_reference(tmp_path, mutation, message):
    good, bad = str(tmp_path / "good.npz"), str(tmp_path / "bad.npz")
    save_deploy(good, CFG, TENSORS)
    rewrite(good, bad, **mutation)
    with pytest.raises(MuNetError, match=message):
        inspect_artifact(bad)
    if oracle.have_ref():  # and the reference's loader rejects the same file
        ok, _ = oracle.ref().load_npz_ok(bad)
        assert not ok


def test_training_payload_keys_are_refused(tmp_path):
    p = str(tmp_path / "m.npz")
    save_deploy(p, CFG, dict(TENSORS, **{"optimizer.state": np.zeros(1, np.float32)}))
    with pytest.raises(MuNetError, match="training/checkpoint payload key"):
        inspect_artifact(p)


def test_missing_and_garbage_files(tmp_path):
    with pytest.raises(MuNetError, match="Unable to open"):
        inspect_artifact(str(tmp_path / "nope.npz"))
    g = tmp_path / "garbage.npz"
    g.write_bytes(b"not a zip archive at all, just bytes" * 4)
    with pytest.raises(MuNetError, match="zip"):
        inspect_artifact(str(g))


def test_json_edge_cases(tmp_path):
    p = str(tmp_path / "m.npz")
    cfg = {"type": "Sequential", "layers": [{"type": "Dropout", "p": 0.25},
                                            {"type": "LayerNorm", "normalized_shape": 4, "eps": 1e-5}]}
    save_deploy(p, cfg, {"1.weight": np.ones(4, np.float32), "1.bias": np.zeros(4, np.float32)})
    got = inspect_artifact(p)["config"]
    assert got["layers"][0]["p"] == 0.25 and abs(got["layers"][1]["eps"] - 1e-5) < 1e-12


def _patch(path, old: bytes, new: bytes, dst):
    data = open(path, "rb").read()
    assert old in data and len(old) == len(new)
    open(dst, "wb").write(data.replace(old, new))


def test_malformed_files_are_refused_not_crashed_on(tmp_path):
    """Truncated headers and size fields that point outside the file: the loader is reached through
    extern "C" entry points that promise never to throw, so every one of these must come back as
    an ordinary load failure."""
    import struct
    good = str(tmp_path / "good.npz")
    save_deploy(good, CFG, TENSORS)
    # 1. an npy header in which nothing follows 'fortran_order:'
    bad = str(tmp_path / "fortran.npz")
    data = open(good, "rb").read()
    i = data.index(b"'fortran_order': False")
    j = data.index(b"\n", i)  # npy headers end with a newline
    data = data[:i] + b"'fortran_order':" + b" " * (j - i - len(b"'fortran_order':")) + data[j:]
    open(bad, "wb").write(data)
    with pytest.raises(MuNetError):
        inspect_artifact(bad)
    # 2. the file cut short at several places
    raw = open(good, "rb").read()
    for cut in (10, 30, len(raw) // 2, len(raw) - 30, len(raw) - 5):
        t = str(tmp_path / f"cut{cut}.npz")
        open(t, "wb").write(raw[:cut])
        with pytest.raises(MuNetError):
            inspect_artifact(t)
    # 3. central-directory fields (entry sizes, local header offsets, directory offset) blown up
    eocd = raw.rindex(b"PK\x05\x06")
    cd_off = struct.unpack_from("<I", raw, eocd + 16)[0]
    for field_off, value in ((20, 0xFFFFFFF0), (24, 0xFFFFFFF0), (42, 0xFFFFFFF0)):
        b = bytearray(raw)
        struct.pack_into("<I", b, cd_off + field_off, value)
        t = str(tmp_path / f"cd{field_off}.npz")
        open(t, "wb").write(bytes(b))
        with pytest.raises(MuNetError):
            inspect_artifact(t)
    b = bytearray(raw)
    struct.pack_into("<I", b, eocd + 16, 0xFFFFFFF0)
    struct.pack_into("<I", b, eocd + 12, 0x20)
    t = str(tmp_path / "eocd.npz")
    open(t, "wb").write(bytes(b))
    with pytest.raises(MuNetError):
        inspect_artifact(t)
    # 4. a shape whose element count wraps around 2^64
    t = str(tmp_path / "shape.npz")
    i = raw.index(b"'shape': (3, 2)")
    b = raw[:i] + b"'shape': (3, 9)" + raw[i + len(b"'shape': (3, 2)"):]
    open(t, "wb").write(b)
    with pytest.raises(MuNetError, match="shorter than its shape"):
        inspect_artifact(t)
