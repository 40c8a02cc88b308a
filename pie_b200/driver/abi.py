"""The runtime <-> driver wire format: a flat, versioned, append-only encoding of the schema of
`driver/schema.py`, the same bytes whether a frame crosses a thread, a process (the shared-memory
control ring of tensor parallelism) or a language boundary (`csrc/include/pie_bridge.h`, generated
from the table below, lets a C / C++ driver read a frame in place without copying).

Frame = 64-byte header + section table + 16-byte aligned sections:

    header   : magic "PIE4", schema version, schema hash (low 64 bits), kind, section count, frame bytes
    section  : {id u32, dtype u32, count u64, offset u64}  (one per non-empty array field)
    payload  : little-endian arrays; strings / nested lists as JSON bytes

Evolution rule: fields are only ever appended (new ids at the end, old ids never renumbered or
retyped); `schema_lock.json` pins the history and `check_append_only()` (run by the tests) refuses a
table that reorders, removes or retypes a locked field. A reader skips section ids it does not know.

Counterpart of driver/bridge/src/schema.rs:44-353 (content, append-only + SCHEMA_HASH),
driver/bridge-macros (the derive that emits the C-ABI readers) and driver/bridge/include/pie_bridge.h.
"""
from __future__ import annotations

import hashlib
import json
import struct
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import numpy as np

from .schema import (CopyDir, CopyRequest, ForwardRequest, ForwardResponse, SamplerKind, SamplerSpec, SlotOutput)

MAGIC = b"PIE4"
SCHEMA_VERSION = 2
KIND_FORWARD_REQUEST, KIND_FORWARD_RESPONSE, KIND_COPY_REQUEST, KIND_DECODE_STEP, KIND_CONTROL = 1, 2, 3, 4, 5
TOKEN_MAGIC = b"PIETFWD1"      # token-only response: magic, u32 count, f32 forward us, f32 total us, then int32 tokens

# dtype codes of sections
U8, I32, I64, F32, U64, JSON = 1, 2, 3, 4, 5, 6
_NP = {U8: np.uint8, I32: np.int32, I64: np.int64, F32: np.float32, U64: np.uint64}
_CNAME = {U8: "uint8_t", I32: "int32_t", I64: "int64_t", F32: "float", U64: "uint64_t", JSON: "char"}

# (struct, field, section id, dtype). APPEND ONLY.
FIELDS: List[Tuple[str, str, int, int]] = [
    ("forward_request", "tokens", 1, I32),
    ("forward_request", "positions", 2, I32),
    ("forward_request", "qo_indptr", 3, I32),
    ("forward_request", "kv_page_indices", 4, I32),
    ("forward_request", "kv_page_indptr", 5, I32),
    ("forward_request", "kv_last_page_lens", 6, I32),
    ("forward_request", "has_user_mask", 7, U8),
    ("forward_request", "mask_runs", 8, I32),             # CSR values: BRLE rows back to back
    ("forward_request", "mask_row_indptr", 9, I32),
    ("forward_request", "logit_masks", 10, I32),          # CSR values: one BRLE per request that has one
    ("forward_request", "slot_req", 11, I32),
    ("forward_request", "slot_row", 12, I32),
    ("forward_request", "sampler_kind", 13, I32),         # SoA of slot_samplers
    ("forward_request", "sampler_temperature", 14, F32),
    ("forward_request", "sampler_top_k", 15, I32),
    ("forward_request", "sampler_top_p", 16, F32),
    ("forward_request", "sampler_min_p", 17, F32),
    ("forward_request", "sampler_seed", 18, I64),
    ("forward_request", "sampler_labels", 19, I32),       # CSR values
    ("forward_request", "sampler_labels_indptr", 20, I32),
    ("forward_request", "spec_counts", 21, I32),
    ("forward_request", "context_ids", 22, U64),
    ("forward_request", "adapter_ids", 23, I64),
    ("forward_request", "flags", 24, I32),                # [single_token_mode, trimmed_pages]
    ("forward_request", "sampler_seed_final", 25, U8),
    ("forward_request", "mask_runs_indptr", 26, I32),
    ("forward_request", "logit_masks_indptr", 27, I32),
    ("forward_request", "logit_masks_present", 28, U8),
    ("forward_response", "slot_kind", 40, I32),
    ("forward_response", "slot_token", 41, I32),
    ("forward_response", "slot_payload", 42, JSON),       # non-token slots: ids / probs / logprobs / entropy / base64 logits
    ("forward_response", "tokens", 43, I32),
    ("forward_response", "timings_us", 44, F32),          # build, h2d, forward, sample, d2h, total
    ("copy_request", "direction", 60, I32),
    ("copy_request", "srcs", 61, I32),
    ("copy_request", "dsts", 62, I32),
    ("decode_step", "meta", 80, I32),                     # [rows, parity]
    ("decode_step", "host_tokens", 81, I32),
    ("decode_step", "src_row", 82, I32),
    ("decode_step", "positions", 83, I32),
    ("decode_step", "kv_lens", 84, I32),
    ("decode_step", "page_indptr", 85, I32),
    ("decode_step", "page_indices", 86, I32),
    ("decode_step", "temperature", 87, F32),
    ("decode_step", "top_k", 88, I32),
    ("decode_step", "top_p", 89, F32),
    ("decode_step", "min_p", 90, F32),
    ("decode_step", "seeds", 91, I64),
    ("control", "json", 100, JSON),                       # cold operations: adapters, health, capabilities, shutdown
    ("forward_response", "spec_accepted", 45, I32),       # accepted drafts per request
    ("forward_request", "rs_slots", 29, I32),             # recurrent-state slot per request
    ("forward_request", "rs_reset", 30, I32),             # 1 = the slot starts from zero in this fire
    ("forward_request", "media_slot", 31, I32),           # media spans: the driver-held clip of each span,
    ("forward_request", "media_src", 32, I32),            # its first encoder-output row,
    ("forward_request", "media_dst", 33, I32),            # the first token row of the batch that takes it,
    ("forward_request", "media_count", 34, I32),          # and the number of rows
]

_SLOT_KINDS = ["token", "distribution", "logits", "logprobs", "entropy", "embedding"]
LOCK = Path(__file__).with_name("schema_lock.json")


def schema_hash() -> str:
    h = hashlib.blake2b(digest_size=16)
    h.update(f"v{SCHEMA_VERSION};".encode())
    for s, f, i, d in FIELDS:
        h.update(f"{s}.{f}:{i}:{d};".encode())
    return h.hexdigest()


def check_append_only(fields=None, lock_path: Path = LOCK) -> None:
    """Raise if the field table reorders, removes, renumbers or retypes anything the lock file pins."""
    fields = FIELDS if fields is None else fields
    locked = [tuple(x) for x in json.loads(lock_path.read_text())["fields"]]
    cur = [tuple(x) for x in fields]
    if cur[:len(locked)] != locked:
        for a, b in zip(locked, cur):
            if a != b:
                raise ValueError(f"wire schema is append-only: locked {a} became {b}")
        raise ValueError("wire schema is append-only: a locked field was removed")
    ids = [i for _, _, i, _ in cur]
    if len(set(ids)) != len(ids):
        raise ValueError("wire schema: duplicate section id")


def write_lock(lock_path: Path = LOCK) -> None:
    lock_path.write_text(json.dumps({"version": SCHEMA_VERSION, "hash": schema_hash(),
                                     "fields": [list(x) for x in FIELDS]}, indent=1) + "\n")


_ID = {(s, f): (i, d) for s, f, i, d in FIELDS}
_BY_ID = {i: (s, f, d) for s, f, i, d in FIELDS}
_HDR = struct.Struct("<4sIQIIQ32x")          # magic, version, hash64, kind, nsections, frame bytes
_SEC = struct.Struct("<IIQQ")


def _frame(kind: int, struct_name: str, values: Dict[str, object]) -> bytes:
    secs, blobs = [], []
    for name, v in values.items():
        if v is None:
            continue
        sid, dt = _ID[(struct_name, name)]
        if dt == JSON:
            raw = json.dumps(v, separators=(",", ":")).encode()
            count = len(raw)
        else:
            arr = np.ascontiguousarray(v, dtype=_NP[dt])
            raw, count = arr.tobytes(), arr.size
        secs.append((sid, dt, count))
        blobs.append(raw)
    off = _HDR.size + _SEC.size * len(secs)
    table, body = [], []
    for (sid, dt, count), raw in zip(secs, blobs):
        pad = (-off) % 16
        body.append(b"\0" * pad)
        off += pad
        table.append(_SEC.pack(sid, dt, count, off))
        body.append(raw)
        off += len(raw)
    hdr = _HDR.pack(MAGIC, SCHEMA_VERSION, int(schema_hash()[:16], 16), kind, len(secs), off)
    return hdr + b"".join(table) + b"".join(body)


def _sections(buf) -> Tuple[int, Dict[str, object]]:
    mv = memoryview(buf)
    magic, ver, h64, kind, nsec, total = _HDR.unpack_from(mv, 0)
    if magic != MAGIC:
        raise ValueError("not a PIE4 frame")
    if ver != SCHEMA_VERSION or h64 != int(schema_hash()[:16], 16):
        raise ValueError(f"wire schema mismatch: frame v{ver}/{h64:016x}, reader v{SCHEMA_VERSION}/{schema_hash()[:16]}")
    if total > len(mv):
        raise ValueError("truncated frame")
    out = {}
    for k in range(nsec):
        sid, dt, count, off = _SEC.unpack_from(mv, _HDR.size + k * _SEC.size)
        if sid not in _BY_ID:
            continue                          # a newer writer's field
        _, name, _ = _BY_ID[sid]
        if dt == JSON:
            out[name] = json.loads(bytes(mv[off:off + count]))
        else:
            out[name] = np.frombuffer(mv, dtype=_NP[dt], count=count, offset=off).copy()
    return kind, out


# ----------------------------------------------------------------------------- forward request
def _csr(rows):
    ptr = np.zeros(len(rows) + 1, np.int32)
    np.cumsum([len(x) for x in rows], out=ptr[1:])
    vals = np.concatenate([np.asarray(x, dtype=np.int32) for x in rows]) if len(rows) and ptr[-1] else np.zeros(0, np.int32)
    return vals, ptr


def _uncsr(vals, ptr):
    return [vals[ptr[i]:ptr[i + 1]].tolist() for i in range(len(ptr) - 1)]


def pack_forward_request(r: ForwardRequest) -> bytes:
    ss = r.slot_samplers
    lab_ptr = np.zeros(len(ss) + 1, np.int32)
    np.cumsum([len(s.labels) for s in ss], out=lab_ptr[1:])
    mr_v, mr_p = (None, None) if r.mask_runs is None else _csr(r.mask_runs)
    lm_v = lm_p = lm_f = None
    if r.logit_masks:
        lm_f = np.asarray([m is not None for m in r.logit_masks], dtype=np.uint8)
        lm_v, lm_p = _csr([m for m in r.logit_masks if m is not None])
    vals = {
        "tokens": r.tokens, "positions": r.positions, "qo_indptr": r.qo_indptr,
        "kv_page_indices": r.kv_page_indices, "kv_page_indptr": r.kv_page_indptr,
        "kv_last_page_lens": r.kv_last_page_lens,
        "has_user_mask": None if r.has_user_mask is None else np.asarray(r.has_user_mask, dtype=np.uint8),
        "mask_runs": mr_v, "mask_runs_indptr": mr_p,
        "mask_row_indptr": r.mask_row_indptr,
        "logit_masks": lm_v, "logit_masks_indptr": lm_p, "logit_masks_present": lm_f,
        "slot_req": r.slot_req, "slot_row": r.slot_row,
        "sampler_kind": [int(s.kind) for s in ss], "sampler_temperature": [s.temperature for s in ss],
        "sampler_top_k": [s.top_k for s in ss], "sampler_top_p": [s.top_p for s in ss],
        "sampler_min_p": [s.min_p for s in ss], "sampler_seed": [s.seed for s in ss],
        "sampler_labels": [int(x) for s in ss for x in s.labels], "sampler_labels_indptr": lab_ptr,
        "sampler_seed_final": [1 if s.seed_final else 0 for s in ss],
        "spec_counts": r.spec_counts, "context_ids": r.context_ids, "adapter_ids": r.adapter_ids,
        "rs_slots": r.rs_slots, "rs_reset": r.rs_reset,
        "media_slot": r.media_slot, "media_src": r.media_src, "media_dst": r.media_dst, "media_count": r.media_count,
        "flags": [1 if r.single_token_mode else 0, int(r.trimmed_pages)],
    }
    return _frame(KIND_FORWARD_REQUEST, "forward_request", vals)


def unpack_forward_request(buf) -> ForwardRequest:
    kind, s = _sections(buf)
    if kind != KIND_FORWARD_REQUEST:
        raise ValueError("not a forward request frame")
    n = len(s.get("sampler_kind", []))
    lab, ptr = s.get("sampler_labels", np.zeros(0, np.int32)), s.get("sampler_labels_indptr", np.zeros(n + 1, np.int32))
    fin = s.get("sampler_seed_final", np.zeros(n, np.uint8))
    samplers = [SamplerSpec(SamplerKind(int(s["sampler_kind"][i])), float(s["sampler_temperature"][i]),
                            int(s["sampler_top_k"][i]), float(s["sampler_top_p"][i]), float(s["sampler_min_p"][i]),
                            int(s["sampler_seed"][i]), tuple(int(x) for x in lab[ptr[i]:ptr[i + 1]]), bool(fin[i]))
                for i in range(n)]
    flags = s.get("flags", np.zeros(2, np.int32))
    e = lambda k, dt: s.get(k, np.zeros(0, dt))
    mask_runs = _uncsr(e("mask_runs", np.int32), s["mask_runs_indptr"]) if "mask_runs_indptr" in s else None
    logit_masks = None
    if "logit_masks_present" in s:
        rows = iter(_uncsr(e("logit_masks", np.int32), s["logit_masks_indptr"]))
        logit_masks = [next(rows) if f else None for f in s["logit_masks_present"]]
    return ForwardRequest(
        tokens=e("tokens", np.int32), positions=e("positions", np.int32), qo_indptr=e("qo_indptr", np.int32),
        kv_page_indices=e("kv_page_indices", np.int32), kv_page_indptr=e("kv_page_indptr", np.int32),
        kv_last_page_lens=e("kv_last_page_lens", np.int32),
        has_user_mask=None if "has_user_mask" not in s else s["has_user_mask"].astype(bool),
        mask_runs=mask_runs, mask_row_indptr=s.get("mask_row_indptr"), logit_masks=logit_masks,
        slot_req=e("slot_req", np.int32), slot_row=e("slot_row", np.int32), slot_samplers=samplers,
        spec_counts=s.get("spec_counts"), context_ids=s.get("context_ids"), adapter_ids=s.get("adapter_ids"),
        rs_slots=s.get("rs_slots"), rs_reset=s.get("rs_reset"),
        media_slot=s.get("media_slot"), media_src=s.get("media_src"), media_dst=s.get("media_dst"),
        media_count=s.get("media_count"),
        single_token_mode=bool(flags[0]), trimmed_pages=int(flags[1]))


# ----------------------------------------------------------------------------- forward response
def pack_forward_response(r: ForwardResponse) -> bytes:
    import base64
    payload = []
    for sl in r.slots:
        if sl.kind == "token":
            payload.append(None)
        else:
            payload.append({"ids": sl.ids, "probs": sl.probs, "logprobs": sl.logprobs, "entropy": sl.entropy,
                            "logits": None if sl.logits is None else base64.b64encode(sl.logits).decode()})
    vals = {"slot_kind": [_SLOT_KINDS.index(sl.kind) for sl in r.slots], "slot_token": [sl.token for sl in r.slots],
            "slot_payload": payload if any(p is not None for p in payload) else None, "tokens": r.tokens,
            "timings_us": [r.t_build_us, r.t_h2d_us, r.t_forward_us, r.t_sample_us, r.t_d2h_us, r.t_total_us],
            "spec_accepted": r.spec_accepted}
    return _frame(KIND_FORWARD_RESPONSE, "forward_response", vals)


def unpack_forward_response(buf) -> ForwardResponse:
    import base64
    kind, s = _sections(buf)
    if kind != KIND_FORWARD_RESPONSE:
        raise ValueError("not a forward response frame")
    kinds, toks = s.get("slot_kind", np.zeros(0, np.int32)), s.get("slot_token", np.zeros(0, np.int32))
    payload = s.get("slot_payload") or [None] * len(kinds)
    slots = []
    for k, t, p in zip(kinds, toks, payload):
        sl = SlotOutput(_SLOT_KINDS[int(k)], token=int(t))
        if p is not None:
            sl.ids, sl.probs, sl.logprobs, sl.entropy = p["ids"], p["probs"], p["logprobs"], p["entropy"]
            sl.logits = None if p["logits"] is None else base64.b64decode(p["logits"])
        slots.append(sl)
    t = s.get("timings_us", np.zeros(6, np.float32))
    return ForwardResponse(slots, s.get("tokens"), *[float(x) for x in t], spec_accepted=s.get("spec_accepted"))


# ----------------------------------------------------------------------------- copy request
def pack_copy_request(r: CopyRequest) -> bytes:
    return _frame(KIND_COPY_REQUEST, "copy_request", {"direction": [int(r.direction)], "srcs": r.srcs, "dsts": r.dsts})


def unpack_copy_request(buf) -> CopyRequest:
    kind, s = _sections(buf)
    if kind != KIND_COPY_REQUEST:
        raise ValueError("not a copy request frame")
    return CopyRequest(CopyDir(int(s["direction"][0])), s.get("srcs", np.zeros(0, np.int32)), s.get("dsts", np.zeros(0, np.int32)))


# ----------------------------------------------------------------------------- pipelined decode step
_STEP_ARRAYS = ("host_tokens", "src_row", "positions", "kv_lens", "page_indptr", "page_indices", "temperature",
                "top_k", "top_p", "min_p", "seeds")


def pack_decode_step(step, parity: int) -> bytes:
    vals = {"meta": [int(step.r), int(parity)]}
    vals.update({k: getattr(step, k) for k in _STEP_ARRAYS})
    return _frame(KIND_DECODE_STEP, "decode_step", vals)


def unpack_decode_step(buf):
    from .executor import CohortStep
    kind, s = _sections(buf)
    if kind != KIND_DECODE_STEP:
        raise ValueError("not a decode step frame")
    dt = {k: _NP[_ID[("decode_step", k)][1]] for k in _STEP_ARRAYS}
    return CohortStep(int(s["meta"][0]), *[s.get(k, np.zeros(0, dt[k])) for k in _STEP_ARRAYS]), int(s["meta"][1])


def pack_tokens(tokens, forward_us: float = 0.0, total_us: float = 0.0) -> bytes:
    t = np.ascontiguousarray(tokens, dtype=np.int32)
    return TOKEN_MAGIC + struct.pack("<Iff", t.size, forward_us, total_us) + t.tobytes()


def is_token_frame(buf) -> bool:
    return bytes(buf[:8]) == TOKEN_MAGIC


def unpack_tokens(buf):
    n, fwd, tot = struct.unpack_from("<Iff", buf, 8)
    return np.frombuffer(buf, dtype=np.int32, count=n, offset=20).copy(), fwd, tot


def pack_control(obj: dict) -> bytes:
    return _frame(KIND_CONTROL, "control", {"json": obj})


def unpack_control(buf) -> dict:
    kind, s = _sections(buf)
    if kind != KIND_CONTROL:
        raise ValueError("not a control frame")
    return s["json"]


def frame_kind(buf) -> int:
    return _HDR.unpack_from(buf, 0)[3]


# ----------------------------------------------------------------------------- C header
def c_header() -> str:
    """`pie_bridge.h`: the frame layout and the section ids for drivers written in C or C++."""
    lines = [
        "/* Generated by pie_b200.driver.abi.c_header(): do not edit. Wire frame of the runtime <-> driver",
        " * channel: 64-byte header, section table, 16-byte aligned little-endian sections. Section ids are",
        " * append-only; skip ids you do not know. */",
        "#ifndef PIE_BRIDGE_H", "#define PIE_BRIDGE_H", "#include <stdint.h>", "#include <string.h>", "",
        f"#define PIE_BRIDGE_SCHEMA_VERSION {SCHEMA_VERSION}u",
        f"#define PIE_BRIDGE_SCHEMA_HASH64 0x{schema_hash()[:16]}ull", "",
        "enum PieFrameKind { PIE_FRAME_FORWARD_REQUEST = 1, PIE_FRAME_FORWARD_RESPONSE = 2, PIE_FRAME_COPY_REQUEST = 3,",
        "                    PIE_FRAME_DECODE_STEP = 4, PIE_FRAME_CONTROL = 5 };",
        "/* A token-only response skips the frame: \"PIETFWD1\", uint32 count, float forward_us, float total_us, int32[count]. */",
        "enum PieSectionType { PIE_U8 = 1, PIE_I32 = 2, PIE_I64 = 3, PIE_F32 = 4, PIE_U64 = 5, PIE_JSON = 6 };", "",
        "typedef struct PieFrameHeader {", "    char magic[4];            /* \"PIE4\" */", "    uint32_t schema_version;",
        "    uint64_t schema_hash64;", "    uint32_t kind;", "    uint32_t num_sections;", "    uint64_t frame_bytes;",
        "    uint8_t reserved[32];", "} PieFrameHeader;", "",
        "typedef struct PieSection {", "    uint32_t id;", "    uint32_t type;", "    uint64_t count;          /* elements (bytes for PIE_JSON) */",
        "    uint64_t offset;         /* from the start of the frame */", "} PieSection;", "",
        "enum PieSectionId {"]
    for st, f, i, d in FIELDS:
        lines.append(f"    PIE_{st.upper()}_{f.upper()} = {i},   /* {_CNAME[d]}[] */")
    lines += ["};", "",
              "/* The section with `id`, or NULL. `frame` must hold header.frame_bytes bytes. */",
              "static inline const PieSection* pie_frame_section(const void* frame, uint32_t id) {",
              "    const PieFrameHeader* h = (const PieFrameHeader*)frame;",
              "    if (memcmp(h->magic, \"PIE4\", 4) != 0 || h->schema_version != PIE_BRIDGE_SCHEMA_VERSION) return 0;",
              "    const PieSection* s = (const PieSection*)((const char*)frame + sizeof(PieFrameHeader));",
              "    for (uint32_t i = 0; i < h->num_sections; ++i)", "        if (s[i].id == id) return &s[i];",
              "    return 0;", "}",
              "static inline const void* pie_section_data(const void* frame, const PieSection* s) {",
              "    return s ? (const char*)frame + s->offset : 0;", "}", "", "#endif", ""]
    return "\n".join(lines)


HEADER_PATH = Path(__file__).resolve().parents[1] / "csrc" / "include" / "pie_bridge.h"
