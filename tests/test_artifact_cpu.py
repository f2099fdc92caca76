"""The weight-container reader on CPU: the structural checks the reference's reader makes
(crates/velox-weights/src/tests.rs:60-121: a valid file opens; ten kinds of damage are refused),
multi-part files, activation policies from `uses`, and bindings turned into views whose bytes
decode to the oracle's values."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from velox_inferer_b200 import ActPolicy, Unsupported
from velox_inferer_b200.artifact import Artifact, ArtifactError, Loader, PAGE

from .artifact_fixture import write_ninfer, write_vi


def test_opens_valid_ninfer(tmp_path):
    a = Artifact.open(write_ninfer(str(tmp_path)))
    assert a.container == "ninfer v3"
    assert len(a.objects) == 3 and len(a.directory["bindings"]) == 3
    assert a.name() == "synthetic"
    assert a.read_object("r.tok")[0] == 768 % 251
    assert a.artifact_id == bytes([7] * 16)


def _set(path, value):
    def mutate(d):
        node = d
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
    return mutate


@pytest.mark.parametrize("name,mutate", [
    ("overlap", _set(("objects", 1, "offset"), 0)),
    ("unaligned tensor", _set(("objects", 1, "offset"), 300)),
    ("part range", _set(("bindings", "text/k", "parts", 0, "range"), [64, 129])),
    ("missing object", _set(("bindings", "text/final_norm", "object"), "nope")),
    ("resource bound as tensor", _set(("bindings", "text/final_norm", "object"), "r.tok")),
    ("unknown root", _set(("extra",), 1)),
    ("velox field in ninfer", _set(("velox",), {})),
    ("bad policy", _set(("uses", 0, "activation_policy"), "A4Only")),
    ("dangling target", _set(("components", "mtp", "target"), "vision")),
    ("length mismatch", _set(("files", 0, "payload_bytes"), 9769)),
    ("no text component", lambda d: d["components"].pop("text")),
    ("use of an unknown parameter", _set(("uses", 0, "parameter"), "text/zz")),
    ("object past the payload", _set(("objects", 2, "bytes"), 9001)),
])
def test_rejects_structural_errors(tmp_path, name, mutate):
    with pytest.raises(ArtifactError):
        Artifact.open(write_ninfer(str(tmp_path), mutate))


def test_rejects_wrong_magic_and_truncation(tmp_path):
    p = write_ninfer(str(tmp_path))
    raw = open(p, "rb").read()
    bad = os.path.join(str(tmp_path), "bad.ninfer")
    open(bad, "wb").write(b"NOTMAGIC" + raw[8:])
    with pytest.raises(ArtifactError):
        Artifact.open(bad)
    cut = os.path.join(str(tmp_path), "cut.ninfer")
    open(cut, "wb").write(raw[:-100])                      # payload shorter than the file table says
    with pytest.raises(ArtifactError):
        Artifact.open(cut)


def test_multi_part_vi_reads_the_same_bytes(tmp_path):
    one, mats = write_vi(str(tmp_path), name="one.vi")
    a = Artifact.open(one)
    many, _ = write_vi(str(tmp_path), part_limit=12 * PAGE, name="many.vi")      # objects split across parts
    b = Artifact.open(many)
    assert a.container == b.container == "velox vi v1"
    assert len(a.files) == 1 and len(b.files) >= 3
    for oid, (_, _, _, _, _, payload) in mats.items():
        assert a.read_object(oid) == payload.tobytes() == b.read_object(oid)
    assert b.format_summary()[0][0] == "nvfp4 / block_scale_k16_m128x4_v1"
    # a part that belongs to another artifact (wrong id in its header) is refused
    part = b.files[1].path
    raw = bytearray(open(part, "rb").read())
    raw[16] ^= 0xFF
    open(part, "wb").write(bytes(raw))
    with pytest.raises(ArtifactError):
        Artifact.open(many)
    with pytest.raises(ArtifactError):                                            # never overwrites
        write_vi(str(tmp_path), name="one.vi")


def test_activation_policies_follow_the_uses(tmp_path):
    path, _ = write_vi(str(tmp_path))
    pol = Artifact.open(path).read_policies()
    assert pol["text/q"] == ActPolicy.allow_a4(600.0)
    assert pol["text/k"] == ActPolicy.allow_a8()           # AllowA4 without a readable divisor
    assert pol["text/v"] == ActPolicy.allow_a8()           # strictest of AllowA4{600} and AllowA8
    assert pol["text/o"] == ActPolicy.allow_a8()
    assert pol["text/down"] == ActPolicy.a16_only()


class HostBackend:
    """Stands in for a device: keeps uploaded bytes as numpy arrays."""

    def __init__(self):
        self.uploads = 0

    def upload_bytes(self, data):
        self.uploads += 1
        return np.asarray(data, dtype=np.uint8).copy()


def test_loader_turns_bindings_into_views_of_one_parent(tmp_path):
    path, mats = write_vi(str(tmp_path))
    ld = Loader(HostBackend(), Artifact.open(path))
    q, k, v = ld.matrix("text/q"), ld.matrix("text/k"), ld.matrix("text/v")
    assert ld.b.uploads == 1 and q.buf is k.buf is v.buf                  # one upload of the shared parent
    assert (q.row_begin, q.rows, k.row_begin, k.rows, v.row_begin, v.rows) == (0, 256, 256, 128, 384, 128)
    assert q.act == ActPolicy.allow_a4(600.0) and k.act == ActPolicy.allow_a8()
    qkv = ld.rows_of(["text/q", "text/k", "text/v"])
    assert (qkv.row_begin, qkv.rows) == (0, 512) and qkv.act == ActPolicy.allow_a8()
    with pytest.raises(Unsupported):
        ld.rows_of(["text/q", "text/v"])                                  # not adjacent
    fmt, _, ofmt, n, kk, payload = mats["w.qkv"]
    got = O.decode_rows(ofmt, np.asarray(k.buf), n, kk, k.row_begin, k.rows)
    want = O.decode_rows(ofmt, payload, n, kk, 256, 128)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    for name, oid in (("text/o", "w.o"), ("text/down", "w.down")):
        view = ld.matrix(name)
        _, _, ofmt, n, kk, payload = mats[oid]
        assert (view.parent_rows, view.k, view.row_begin, view.rows) == (n, kk, 0, n)
        assert np.array_equal(np.asarray(view.buf), payload)


def test_loader_refuses_mis_sized_and_unknown_objects(tmp_path):
    def shrink(d):
        d["objects"][0]["shape"] = [512, 320]              # bytes no longer match the layout
    path, _ = write_vi(str(tmp_path), mutate=shrink, name="a.vi")
    from velox_inferer_b200 import ShapeError
    with pytest.raises(ShapeError):
        Loader(HostBackend(), Artifact.open(path)).matrix("text/q")

    def rename(d):
        d["objects"][1]["format"] = "q8_g32_fp16"
        d["objects"][1]["layout"] = "row_split_k128_v1"
    path, _ = write_vi(str(tmp_path), mutate=rename, name="b.vi")
    with pytest.raises(Unsupported):
        Loader(HostBackend(), Artifact.open(path)).matrix("text/o")

    def ragged(d):
        d["bindings"]["text/k"]["parts"][0]["range"] = [256 * 256 + 5, 384 * 256]
    path, _ = write_vi(str(tmp_path), mutate=ragged, name="c.vi")
    with pytest.raises(Unsupported):
        Loader(HostBackend(), Artifact.open(path)).matrix("text/k")
