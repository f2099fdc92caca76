"""Builds small weight containers for the reader's tests: a ninfer v3 file with the structure the
reference's own reader tests use (crates/velox-weights/src/tests.rs:22-58), and a velox .vi whose
tensors are real NVFP4 / FP8-row / Q4_K matrices made by the oracle's constructors, with bindings
(whole objects and row ranges), uses carrying activation policies, and a divisor auxiliary."""
import json
import os
import struct

import numpy as np

from oracle import oracle as O
from velox_inferer_b200.artifact import NINFER_ENTRY_MAGIC, PAGE, align_up, write_container


def ninfer_directory():
    return {
        "components": {
            "text": {"config": {"architectures": ["Qwen3_5ForCausalLM"]}, "resources": {"tokenizer.json": "r.tok"}},
            "mtp": {"config": {"architectures": ["Qwen3_5MTP"]}, "target": "text"},
        },
        "objects": [
            {"id": "w.qk", "kind": "tensor", "shape": [8, 16], "format": "bf16", "layout": "contiguous_le_v1",
             "offset": 0, "bytes": 256},
            {"id": "w.norm", "kind": "tensor", "shape": [16], "format": "fp32", "layout": "contiguous_le_v1",
             "offset": 512, "bytes": 64},
            {"id": "r.tok", "kind": "resource", "encoding": "raw_bytes_v1", "offset": 768, "bytes": 9000},
        ],
        "bindings": {
            "text/q": {"parts": [{"object": "w.qk", "range": [0, 64]}]},
            "text/k": {"parts": [{"object": "w.qk", "range": [64, 128]}]},
            "text/final_norm": {"object": "w.norm"},
        },
        "uses": [{"parameter": "text/q", "input": "text/x", "activation_policy": "AllowA8"}],
        "files": [{"path": None, "payload_bytes": 768 + 9000}],
        "metadata": {"name": "synthetic"},
    }


def write_ninfer(dirpath, mutate=None):
    """Single-file ninfer v3 artifact, payload bytes i % 251, framed by hand (json_bytes = the exact
    JSON length, zero padding up to the page)."""
    d = ninfer_directory()
    if mutate:
        mutate(d)
    blob = json.dumps(d).encode()
    raw = NINFER_ENTRY_MAGIC + struct.pack("<Q", len(blob)) + bytes([7] * 16) + blob
    raw += b"\0" * (align_up(len(raw), PAGE) - len(raw))
    raw += bytes(i % 251 for i in range(768 + 9000))
    p = os.path.join(dirpath, "model.ninfer")
    with open(p, "wb") as f:
        f.write(raw)
    return p


def matrices():
    """name -> (container format, layout, oracle format, n, k, payload bytes)."""
    rng = np.random.default_rng(17)

    def w(n, k):
        return (rng.standard_normal((n, k)) * 0.02).astype(np.float32)

    return {
        "w.qkv": ("nvfp4", "block_scale_k16_m128x4_v1", O.FMT_NVFP4, 512, 256, O.encode_nvfp4_rne(w(512, 256))),
        "w.o": ("fp8_e4m3fn_row_bf16", "row_scale_v1", O.FMT_FP8, 96, 384, O.encode_fp8_row(w(96, 384))),
        "w.down": ("ggml_q4_k", "ggml_block_v1", O.FMT_Q4K, 64, 512, O.encode_q4k(w(64, 512))),
    }


def write_vi(dirpath, part_limit=None, mutate=None, name="model.vi"):
    """A .vi with the three tensor formats. Returns (path, matrices)."""
    mats = matrices()
    objects, blobs, off = [], [], 0
    for oid, (fmt, layout, _, n, k, payload) in mats.items():
        off = align_up(off, 256)
        objects.append({"id": oid, "kind": "tensor", "shape": [n, k], "format": fmt, "layout": layout,
                        "offset": off, "bytes": int(payload.size)})
        blobs.append((off, payload.tobytes()))
        off += payload.size
    off = align_up(off, 256)
    objects.append({"id": "aux.div", "kind": "tensor", "shape": [1], "format": "fp32", "layout": "contiguous_le_v1",
                    "offset": off, "bytes": 4})
    blobs.append((off, struct.pack("<f", 600.0)))
    off += 4
    objects.append({"id": "r.tok", "kind": "resource", "encoding": "raw_bytes_v1", "offset": off, "bytes": 100})
    blobs.append((off, bytes(range(100))))
    total = off + 100
    image = bytearray(total)
    for o, bts in blobs:
        image[o:o + len(bts)] = bts
    k = 256
    d = {
        "components": {"text": {"config": {"hidden_size": 256}, "resources": {"tokenizer.json": "r.tok"}}},
        "objects": objects,
        "bindings": {
            "text/q": {"parts": [{"object": "w.qkv", "range": [0, 256 * k]}]},
            "text/k": {"parts": [{"object": "w.qkv", "range": [256 * k, 384 * k]}]},
            "text/v": {"parts": [{"object": "w.qkv", "range": [384 * k, 448 * k]}, {"object": "w.qkv", "range": [448 * k, 512 * k]}]},
            "text/o": {"object": "w.o"},
            "text/down": {"object": "w.down"},
        },
        "uses": [
            {"parameter": "text/q", "input": "text/x", "activation_policy": "AllowA4",
             "auxiliaries": {"activation_input_divisor": {"object": "aux.div"}}},
            {"parameter": "text/k", "input": "text/x", "activation_policy": "AllowA4"},       # no divisor: A8
            {"parameter": "text/v", "input": "text/x", "activation_policy": "AllowA4",
             "auxiliaries": {"activation_input_divisor": {"object": "aux.div"}}},
            {"parameter": "text/v", "input": "text/y", "activation_policy": "AllowA8"},       # strictest of two uses
            {"parameter": "text/o", "input": "text/a", "activation_policy": "AllowA8"},
            {"parameter": "text/down", "input": "text/h"},                                    # no policy: A16Only
        ],
        "metadata": {"name": "three-formats"},
        "velox": {"format_version": 1, "source_container": "none", "source_artifact_id": "00" * 16},
    }
    if mutate:
        mutate(d)
    path = os.path.join(dirpath, name)
    kw = {} if part_limit is None else {"part_limit": part_limit}
    write_container(path, d, total, lambda at, n: bytes(image[at:at + n]), container="velox vi v1", **kw)
    return path, mats
