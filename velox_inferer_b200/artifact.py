"""Reader of velox weight containers (``.vi`` v1 and ``.ninfer`` v3) for the tensor formats this
kernel set executes, and the loader that turns bindings into ``WeightView`` objects.

Mirrors the reference's ``velox-weights`` crate and the weight loader of its model crate:

* ``Artifact.open``: framing, file table and part headers, object order / alignment / overlap, and
  every binding, use, resource and component reference
  (crates/velox-weights/src/lib.rs:167-240 ``open``, :242-316 ``parse_files``, :318-394
  ``parse_objects``, :396-520 ``check_binding`` / ``check_references``; docs/weights.md:14-25);
* ``read_range`` / ``read_object``: logical payload bytes across parts (lib.rs:547-580);
* ``read_policies``: ``uses[].activation_policy`` with the ``activation_input_divisor`` auxiliary,
  strictest over a parameter's uses, ``A16Only`` for anything unreadable
  (crates/velox-models/src/qwen3_5/weights.rs:291-315);
* ``Loader.binding`` / ``parent`` / ``matrix`` / ``rows_of``: one upload per parent object, row
  views for whole-row ranges, adjacent views merged (weights.rs:318-385, 520-575).

``write_container`` writes the same framing (lib.rs:640-745) and is what the tests build their
fixtures with. Pure host code: nothing here touches a kernel."""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from .errors import ShapeError, Unsupported
from .weights import ActPolicy, WeightFormat, WeightView

NINFER_ENTRY_MAGIC = b"NINFER\x00\x03"
NINFER_PART_MAGIC = b"NINPRT\x00\x03"
VI_ENTRY_MAGIC = b"VELOXVI\x01"
VI_PART_MAGIC = b"VELOXPT\x01"
HEADER = 32
PAGE = 4096
DEFAULT_PART_LIMIT = 32_000_000_000
DRAFTER_COMPONENTS = ("dflash2", "dspine")

_ROOT_FIELDS = ("components", "objects", "bindings", "uses", "files", "metadata", "provenance")


class ArtifactError(ValueError):
    """``Error::Format``: the file is not a valid artifact."""


def _bad(msg: str):
    raise ArtifactError(f"invalid artifact: {msg}")


def align_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def _uint(v, what: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        _bad(f"{what} must be a non-negative integer")
    return v


def _text(o: dict, key: str, what: str) -> str:
    s = o.get(key)
    if not isinstance(s, str) or not s or "\0" in s:
        _bad(f"{what}.{key} must be a non-empty string")
    return s


@dataclass(frozen=True)
class Object:
    """One entry of the directory's ``objects``: a tensor (shape, format, layout) or a resource."""

    id: str
    kind: str                      # "tensor" | "resource"
    offset: int                    # byte offset in the logical payload
    bytes: int
    shape: Tuple[int, ...] = ()
    format: str = ""
    layout: str = ""
    encoding: str = ""

    def elements(self) -> Optional[int]:
        if self.kind != "tensor":
            return None
        n = 1
        for d in self.shape:
            n *= d
        return n


@dataclass(frozen=True)
class FileEntry:
    path: str
    payload_start: int             # byte offset of this file's payload within the file
    payload_bytes: int
    logical_start: int             # start of this file's slice of the logical payload


def _read_header(path: str) -> bytes:
    with open(path, "rb") as f:
        h = f.read(HEADER)
    if len(h) != HEADER:
        raise ArtifactError(f"{path}: shorter than its header")
    return h


class Artifact:
    """An opened container: the verbatim JSON directory, the file table and the object index."""

    def __init__(self, path, container, artifact_id, directory, files, objects):
        self.path, self.container, self.artifact_id = path, container, artifact_id
        self.directory, self.files, self.objects = directory, files, objects
        self._index = {o.id: i for i, o in enumerate(objects)}

    # ---- open -------------------------------------------------------------------------------
    @staticmethod
    def open(path: str) -> "Artifact":
        path = os.fspath(path)
        h = _read_header(path)
        if h[:8] == NINFER_ENTRY_MAGIC:
            container = "ninfer v3"
        elif h[:8] == VI_ENTRY_MAGIC:
            container = "velox vi v1"
        else:
            _bad(f"unknown magic {h[:8].hex()}")
        json_bytes = struct.unpack("<Q", h[8:16])[0]
        if json_bytes == 0 or json_bytes > 1 << 32:
            _bad(f"json_bytes {json_bytes} out of range")
        artifact_id = h[16:32]
        with open(path, "rb") as f:
            f.seek(HEADER)
            raw = f.read(json_bytes)
        if len(raw) != json_bytes:
            raise ArtifactError(f"{path}: directory is cut short")
        try:
            directory = json.loads(raw.decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            _bad(f"directory JSON: {e}")
        if not isinstance(directory, dict):
            _bad("directory is not a JSON object")
        entry_payload_start = align_up(HEADER + json_bytes, PAGE)
        allowed = _ROOT_FIELDS + (("velox",) if container == "velox vi v1" else ())
        for k in directory:
            if k not in allowed:
                _bad(f"unknown root field '{k}'")
        files = Artifact._parse_files(path, container, artifact_id, directory, entry_payload_start)
        payload_bytes = sum(f.payload_bytes for f in files)
        objects = Artifact._parse_objects(directory, payload_bytes)
        a = Artifact(path, container, artifact_id, directory, files, objects)
        a._check_references()
        return a

    @staticmethod
    def _parse_files(path, container, artifact_id, directory, entry_payload_start) -> List[FileEntry]:
        lst = directory.get("files")
        if not isinstance(lst, list) or not lst:
            _bad("files must be a non-empty array")
        base = os.path.dirname(path) or "."
        part_magic = NINFER_PART_MAGIC if container == "ninfer v3" else VI_PART_MAGIC
        out, logical, seen = [], 0, []
        for i, item in enumerate(lst):
            if not isinstance(item, dict):
                _bad(f"files[{i}] is not an object")
            payload_bytes = _uint(item.get("payload_bytes"), f"files[{i}].payload_bytes")
            if payload_bytes == 0:
                _bad(f"files[{i}].payload_bytes must be positive")
            if i == 0:
                if "path" not in item or item["path"] is not None:
                    _bad("files[0].path must be null")
                file_path, payload_start = path, entry_payload_start
            else:
                name = _text(item, "path", f"files[{i}]")
                if "/" in name or "\\" in name or name in (".", "..") or name in seen:
                    _bad(f"files[{i}].path '{name}' is not a unique sibling file name")
                seen.append(name)
                file_path = os.path.join(base, name)
                try:
                    h = _read_header(file_path)
                except OSError as e:
                    raise ArtifactError(f"{file_path}: {e}") from None
                if h[:8] != part_magic or struct.unpack("<Q", h[8:16])[0] != i or h[16:32] != artifact_id:
                    _bad(f"{file_path} is not part {i} of this artifact")
                payload_start = PAGE
            length = os.path.getsize(file_path)
            if length != payload_start + payload_bytes:
                _bad(f"{file_path} is {length} bytes, directory says {payload_start + payload_bytes}")
            out.append(FileEntry(file_path, payload_start, payload_bytes, logical))
            logical += payload_bytes
        return out

    @staticmethod
    def _parse_objects(directory, payload_bytes) -> List[Object]:
        lst = directory.get("objects")
        if not isinstance(lst, list) or not lst:
            _bad("objects must be a non-empty array")
        out: List[Object] = []
        ids = set()
        for i, item in enumerate(lst):
            what = f"objects[{i}]"
            if not isinstance(item, dict):
                _bad(f"{what} is not an object")
            oid = _text(item, "id", what)
            offset = _uint(item.get("offset"), f"{what}.offset")
            nbytes = _uint(item.get("bytes"), f"{what}.bytes")
            kind = item.get("kind")
            if kind == "tensor":
                shape = item.get("shape")
                if not isinstance(shape, list) or len(shape) > 16:
                    _bad(f"{what}.shape must be an array of rank 0..16")
                for d in shape:
                    if isinstance(d, bool) or not isinstance(d, int) or d <= 0:
                        _bad(f"{what}.shape has a non-positive dimension")
                fmt, layout = _text(item, "format", what), _text(item, "layout", what)
                if offset % 256 != 0:
                    _bad(f"tensor {oid} offset {offset} is not 256-byte aligned")
                obj = Object(oid, "tensor", offset, nbytes, tuple(shape), fmt, layout)
            elif kind == "resource":
                obj = Object(oid, "resource", offset, nbytes, encoding=_text(item, "encoding", what))
            else:
                _bad(f"{what}.kind {kind!r} is not tensor or resource")
            if nbytes == 0 or offset + nbytes > payload_bytes:
                _bad(f"object {oid} [{offset}, +{nbytes}) is outside the payload")
            if out and offset < out[-1].offset + out[-1].bytes:
                _bad(f"object {oid} overlaps or precedes {out[-1].id}")
            if oid in ids:
                _bad(f"duplicate object id {oid}")
            ids.add(oid)
            out.append(obj)
        return out

    def object(self, oid: str) -> Optional[Object]:
        i = self._index.get(oid)
        return None if i is None else self.objects[i]

    def _tensor(self, oid, what: str) -> Object:
        o = self.object(oid) if isinstance(oid, str) else None
        if o is None:
            _bad(f"{what} references missing object '{oid}'")
        if o.kind != "tensor":
            _bad(f"{what} references resource '{oid}' where a tensor is required")
        return o

    def _check_binding(self, b, what: str) -> None:
        if not isinstance(b, dict):
            _bad(f"{what} is not an object")
        has_obj, parts = "object" in b, b.get("parts")
        if has_obj and "parts" not in b:
            self._tensor(b["object"] if isinstance(b["object"], str) else "", what)
        elif not has_obj and isinstance(parts, list) and parts:
            for j, p in enumerate(parts):
                pw = f"{what}.parts[{j}]"
                oid = p.get("object", "") if isinstance(p, dict) else ""
                elements = self._tensor(oid, pw).elements()
                r = p.get("range") if isinstance(p, dict) else None
                if (not isinstance(r, list) or len(r) != 2
                        or any(isinstance(v, bool) or not isinstance(v, int) or v < 0 for v in r)):
                    _bad(f"{pw}.range must be [begin, end)")
                if not (r[0] < r[1] <= elements):
                    _bad(f"{pw}.range [{r[0]}, {r[1]}) outside 0..{elements}")
        else:
            _bad(f"{what} must have exactly one of object / non-empty parts")

    def _check_references(self) -> None:
        d = self.directory
        bindings = d.get("bindings")
        if not isinstance(bindings, dict):
            _bad("bindings must be an object")
        for name, b in bindings.items():
            self._check_binding(b, f"binding '{name}'")
        uses = d.get("uses")
        if not isinstance(uses, list):
            _bad("uses must be an array")
        seen = set()
        for i, u in enumerate(uses):
            what = f"uses[{i}]"
            if not isinstance(u, dict):
                _bad(f"{what} is not an object")
            param, inp = _text(u, "parameter", what), _text(u, "input", what)
            if param not in bindings:
                _bad(f"{what} names unknown parameter '{param}'")
            if (param, inp) in seen:
                _bad(f"{what} repeats ({param}, {inp})")
            seen.add((param, inp))
            if "activation_policy" in u and u["activation_policy"] not in ("A16Only", "AllowA8", "AllowA4"):
                _bad(f"{what}.activation_policy {u['activation_policy']!r} is not A16Only/AllowA8/AllowA4")
            aux = u.get("auxiliaries")
            if isinstance(aux, dict):
                for role, b in aux.items():
                    self._check_binding(b, f"{what}.auxiliaries.{role}")
        comps = d.get("components")
        if not isinstance(comps, dict):
            _bad("components must be an object")
        drafter_only = bool(comps) and all(k in DRAFTER_COMPONENTS for k in comps)
        if "text" not in comps and not drafter_only:
            _bad("components must include 'text'")
        for cid, c in comps.items():
            if not isinstance(c, dict) or not isinstance(c.get("config"), dict):
                _bad(f"component '{cid}' needs a config object")
            t = c.get("target")
            if isinstance(t, str) and t not in comps:
                _bad(f"component '{cid}' targets missing component '{t}'")
            res = c.get("resources")
            if isinstance(res, dict):
                for role, rid in res.items():
                    o = self.object(rid) if isinstance(rid, str) else None
                    if o is None or o.kind != "resource":
                        _bad(f"component '{cid}' resource '{role}' is not a resource object")

    # ---- payload ------------------------------------------------------------------------------
    def payload_bytes(self) -> int:
        return sum(f.payload_bytes for f in self.files)

    def name(self) -> Optional[str]:
        md = self.directory.get("metadata")
        n = md.get("name") if isinstance(md, dict) else None
        return n if isinstance(n, str) else None

    def read_range(self, offset: int, length: int) -> bytes:
        """Logical payload bytes [offset, offset + length), crossing files as needed."""
        end = offset + length
        if offset < 0 or length < 0 or end > self.payload_bytes():
            _bad(f"read [{offset}, +{length}) outside payload")
        out = bytearray(length)
        for f in self.files:
            a, b = max(offset, f.logical_start), min(end, f.logical_start + f.payload_bytes)
            if a >= b:
                continue
            with open(f.path, "rb") as fh:
                fh.seek(f.payload_start + (a - f.logical_start))
                chunk = fh.read(b - a)
            if len(chunk) != b - a:
                raise ArtifactError(f"{f.path}: payload is cut short")
            out[a - offset:b - offset] = chunk
        return bytes(out)

    def read_object(self, oid: str) -> bytes:
        o = self.object(oid)
        if o is None:
            _bad(f"no object '{oid}'")
        return self.read_range(o.offset, o.bytes)

    def format_summary(self) -> List[Tuple[str, int, int]]:
        """(format / layout, objects, bytes) over the objects, largest first."""
        m: Dict[str, List[int]] = {}
        for o in self.objects:
            key = f"{o.format} / {o.layout}" if o.kind == "tensor" else f"resource / {o.encoding}"
            e = m.setdefault(key, [0, 0])
            e[0] += 1
            e[1] += o.bytes
        return sorted(((k, n, b) for k, (n, b) in m.items()), key=lambda e: -e[2])

    # ---- activation policies ----------------------------------------------------------------
    def read_policies(self) -> Dict[str, ActPolicy]:
        """Activation policy per parameter (weights.rs:291-315)."""
        out: Dict[str, ActPolicy] = {}
        for u in self.directory.get("uses", []):
            param = u.get("parameter") if isinstance(u, dict) else None
            if not isinstance(param, str):
                continue
            divisor = None
            try:
                oid = u["auxiliaries"]["activation_input_divisor"]["object"]
                raw = self.read_object(oid)
                if len(raw) >= 4:
                    v = struct.unpack("<f", raw[:4])[0]
                    if v == v and v not in (float("inf"), float("-inf")) and v > 0.0:
                        divisor = v
            except (KeyError, TypeError, ArtifactError):
                divisor = None
            pol = u.get("activation_policy")
            if pol == "AllowA4" and divisor is not None:
                p = ActPolicy.allow_a4(divisor)
            elif pol in ("AllowA4", "AllowA8"):
                p = ActPolicy.allow_a8()
            else:
                p = ActPolicy.a16_only()
            out[param] = out[param].meet(p) if param in out else p
        return out


class Loader:
    """Bindings -> ``WeightView`` on a backend, one upload per parent object
    (crates/velox-models/src/qwen3_5/weights.rs:262-385, 520-575)."""

    def __init__(self, backend, art: Artifact):
        self.b, self.art = backend, art
        self.parents: List = []                                   # device buffers, one per uploaded object
        self._index: Dict[str, Tuple[int, WeightFormat, int, int]] = {}
        self.policies = art.read_policies()
        self.bytes = 0

    def binding(self, name: str) -> Tuple[str, Optional[Tuple[int, int]]]:
        """(object id, element range) of a binding that is a whole object or contiguous parts."""
        b = self.art.directory["bindings"].get(name)
        if b is None:
            raise ShapeError(f"artifact has no binding '{name}'")
        if isinstance(b.get("object"), str):
            return b["object"], None
        oid, rng = "", None
        for p in b["parts"]:
            pid, (a, e) = p["object"], p["range"]
            if rng is None:
                oid, rng = pid, (a, e)
            elif pid == oid and a == rng[1]:
                rng = (rng[0], e)                                 # consecutive parts of one parent merge
            else:
                raise Unsupported(f"binding '{name}' gathers non-contiguous parts")
        return oid, rng

    def parent(self, oid: str) -> Tuple[int, WeightFormat, int, int]:
        """Uploads parent ``oid`` once; (slot, format, n, k)."""
        if oid in self._index:
            return self._index[oid]
        obj = self.art.object(oid)
        if obj is None:
            raise ShapeError(f"missing object {oid}")
        if obj.kind != "tensor" or len(obj.shape) != 2:
            raise ShapeError(f"object {oid} is not a matrix: {obj}")
        fmt = WeightFormat.from_names(obj.format, obj.layout)
        n, k = obj.shape
        fmt.check_shape(n, k)
        raw = self.art.read_object(oid)
        if len(raw) != fmt.payload_bytes(n, k):
            raise ShapeError(f"object {oid}: {len(raw)} bytes, layout implies {fmt.payload_bytes(n, k)}")
        import numpy as np

        self.parents.append(self.b.upload_bytes(np.frombuffer(raw, dtype=np.uint8).copy()))
        self.bytes += len(raw)
        self._index[oid] = (len(self.parents) - 1, fmt, n, k)
        return self._index[oid]

    def policy(self, name: str) -> ActPolicy:
        return self.policies.get(name, ActPolicy.a16_only())

    def matrix(self, name: str) -> WeightView:
        oid, rng = self.binding(name)
        slot, fmt, n, k = self.parent(oid)
        if rng is None:
            row_begin, rows = 0, n
        else:
            a, e = rng
            if a % k != 0 or e % k != 0:
                raise Unsupported(f"binding '{name}' range [{a},{e}) is not whole rows of {oid}")
            row_begin, rows = a // k, (e - a) // k
        return WeightView(self.parents[slot], fmt, n, k, row_begin, rows, self.policy(name))

    def rows_of(self, names: Sequence[str]) -> WeightView:
        """Concatenation of row views that are adjacent in one parent, as one view."""
        acc: Optional[WeightView] = None
        for name in names:
            d = self.matrix(name)
            if acc is None:
                acc = d
            elif acc.buf is d.buf and acc.row_begin + acc.rows == d.row_begin:
                acc = WeightView(acc.buf, acc.format, acc.parent_rows, acc.k, acc.row_begin, acc.rows + d.rows,
                                 acc.act.meet(d.act))
            else:
                raise Unsupported(f"{list(names)} are not adjacent rows of one parent")
        return acc


def write_container(out: str, directory: dict, payload_bytes: int, fill: Callable[[int, int], bytes],
                    container: str = "velox vi v1", part_limit: int = DEFAULT_PART_LIMIT,
                    artifact_id: bytes = b"\x07" * 16) -> None:
    """Writes an artifact whose directory is ``directory`` (its ``files`` table is rebuilt) and whose
    logical payload is ``payload_bytes`` bytes produced by ``fill(offset, length)`` in increasing
    offsets. Parts are renamed into place first, the entry last, so a visible entry always has its
    parts; an existing ``out`` is never overwritten (lib.rs:640-745)."""
    if os.path.exists(out):
        _bad(f"{out} already exists")
    entry_magic, part_magic = ((NINFER_ENTRY_MAGIC, NINFER_PART_MAGIC) if container == "ninfer v3"
                               else (VI_ENTRY_MAGIC, VI_PART_MAGIC))
    name = os.path.basename(out)
    directory = dict(directory)
    reserve = PAGE - HEADER
    while True:   # reserve JSON space, lay out files, grow the reservation until the directory fits
        entry_start = align_up(HEADER + reserve, PAGE)
        if part_limit <= entry_start + PAGE:
            _bad("part limit too small")
        entry_cap = (part_limit - entry_start) // PAGE * PAGE
        part_cap = (part_limit - PAGE) // PAGE * PAGE
        sizes = [min(payload_bytes, entry_cap)]
        left = payload_bytes - sizes[0]
        while left > 0:
            sizes.append(min(left, part_cap))
            left -= sizes[-1]
        directory["files"] = [{"path": None if i == 0 else f"{name}.part-{i:04d}", "payload_bytes": b}
                              for i, b in enumerate(sizes)]
        blob = json.dumps(directory, separators=(",", ":")).encode("utf-8")
        if len(blob) <= reserve:
            break
        reserve = align_up(len(blob) + HEADER, PAGE) - HEADER
    base = os.path.dirname(out) or "."
    written = []
    try:
        logical = 0
        for i, nbytes in enumerate(sizes):
            final = out if i == 0 else os.path.join(base, f"{name}.part-{i:04d}")
            tmp = final + ".tmp-velox"
            written.append((tmp, final))
            with open(tmp, "wb") as f:
                if i == 0:
                    head = entry_magic + struct.pack("<Q", reserve) + artifact_id + blob
                    head += b" " * (HEADER + reserve - len(head))
                    head += b"\0" * (align_up(HEADER + reserve, PAGE) - len(head))
                else:
                    head = part_magic + struct.pack("<Q", i) + artifact_id
                    head += b"\0" * (PAGE - len(head))
                f.write(head)
                done = 0
                while done < nbytes:
                    n = min(nbytes - done, 64 << 20)
                    chunk = fill(logical + done, n)
                    assert len(chunk) == n
                    f.write(chunk)
                    done += n
            logical += nbytes
        for tmp, final in reversed(written):
            os.rename(tmp, final)
    except BaseException:
        for tmp, _ in written:
            if os.path.exists(tmp):
                os.remove(tmp)
        raise
