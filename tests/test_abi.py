"""The flat wire format of the runtime <-> driver channel: round trips, schema hash, append-only lock,
generated C header. Model: the schema tests of driver/bridge/src/schema.rs."""
import dataclasses
import subprocess

import numpy as np
import pytest

from pie_b200.driver import abi
from pie_b200.driver.schema import (CopyDir, CopyRequest, ForwardRequest, ForwardResponse, SamplerKind, SamplerSpec,
                                    SlotOutput)


def _req():
    i32 = lambda *a: np.asarray(a, dtype=np.int32)
    return ForwardRequest(
        tokens=i32(5, 6, 7, 8), positions=i32(0, 1, 2, 9), qo_indptr=i32(0, 3, 4), kv_page_indices=i32(2, 3, 7),
        kv_page_indptr=i32(0, 2, 3), kv_last_page_lens=i32(3, 10), has_user_mask=np.asarray([True, False]),
        mask_runs=[[0, 1], [0, 2], [1, 1, 1]], mask_row_indptr=i32(0, 3, 3), logit_masks=[None, [3, 5, 100]],
        slot_req=i32(0, 1), slot_row=i32(2, 3),
        slot_samplers=[SamplerSpec(SamplerKind.TOP_P, 0.7, 0, 0.9, 0.0, 1234567890123, (), True),
                       SamplerSpec(SamplerKind.LOGPROBS, labels=(4, 9))],
        spec_counts=i32(0, 1), context_ids=np.asarray([11, 2 ** 40], dtype=np.uint64), adapter_ids=np.asarray([-1, 3]),
        single_token_mode=False, trimmed_pages=2)


def _same(a, b):
    for f in dataclasses.fields(a):
        x, y = getattr(a, f.name), getattr(b, f.name)
        if isinstance(x, np.ndarray):
            assert y is not None and np.array_equal(x, y), f.name
        elif isinstance(x, list) and x and dataclasses.is_dataclass(x[0]):
            assert len(x) == len(y)
            for p, q in zip(x, y):
                _same(p, q)
        elif isinstance(x, float):
            assert x == pytest.approx(y), f.name
        elif isinstance(x, (list, tuple)):
            assert list(x) == list(y), f.name
        else:
            assert x == y, f.name


def test_forward_request_round_trip():
    r = _req()
    buf = abi.pack_forward_request(r)
    assert buf[:4] == b"PIE4"
    _same(r, abi.unpack_forward_request(buf))


def test_minimal_request_round_trip():
    r = dataclasses.replace(_req(), has_user_mask=None, mask_runs=None, mask_row_indptr=None, logit_masks=None,
                            spec_counts=None, context_ids=None, adapter_ids=None, single_token_mode=True, trimmed_pages=0)
    out = abi.unpack_forward_request(abi.pack_forward_request(r))
    _same(r, out)
    assert out.mask_runs is None and out.logit_masks is None and out.spec_counts is None


def test_response_and_copy_round_trip():
    resp = ForwardResponse([SlotOutput("token", token=42),
                            SlotOutput("distribution", ids=[1, 2], probs=[0.75, 0.25]),
                            SlotOutput("logits", logits=b"\x00\x01\x02\x03"),
                            SlotOutput("entropy", entropy=1.5)],
                           np.asarray([42], dtype=np.int32), 1.0, 2.0, 3.0, 4.0, 5.0, 15.0)
    _same(resp, abi.unpack_forward_response(abi.pack_forward_response(resp)))
    c = CopyRequest(CopyDir(0), np.asarray([1, 2], np.int32), np.asarray([5, 6], np.int32))
    _same(c, abi.unpack_copy_request(abi.pack_copy_request(c)))


def test_sections_are_aligned_and_frame_kind_checked():
    buf = abi.pack_forward_request(_req())
    _, _, _, kind, nsec, total = abi._HDR.unpack_from(buf, 0)
    assert kind == abi.KIND_FORWARD_REQUEST and total == len(buf)
    for k in range(nsec):
        _, _, _, off = abi._SEC.unpack_from(buf, abi._HDR.size + k * abi._SEC.size)
        assert off % 16 == 0
    with pytest.raises(ValueError):
        abi.unpack_copy_request(buf)
    with pytest.raises(ValueError):
        abi.unpack_forward_request(b"XXXX" + buf[4:])
    bad = bytearray(buf)
    bad[8] ^= 0xFF                                   # another schema hash
    with pytest.raises(ValueError, match="schema mismatch"):
        abi.unpack_forward_request(bytes(bad))


def test_schema_is_append_only(tmp_path):
    abi.check_append_only()                          # the committed lock against the live table
    import json
    assert json.loads(abi.LOCK.read_text())["hash"] == abi.schema_hash() or \
        len(json.loads(abi.LOCK.read_text())["fields"]) < len(abi.FIELDS)
    abi.check_append_only(abi.FIELDS + [("forward_request", "new_field", 99, abi.I32)])
    with pytest.raises(ValueError, match="append-only"):
        abi.check_append_only(abi.FIELDS[1:])
    retyped = list(abi.FIELDS)
    retyped[0] = (retyped[0][0], retyped[0][1], retyped[0][2], abi.I64)
    with pytest.raises(ValueError, match="append-only"):
        abi.check_append_only(retyped)
    with pytest.raises(ValueError, match="duplicate"):
        abi.check_append_only(abi.FIELDS + [("forward_request", "dup", 1, abi.I32)])


def test_c_header_is_current_and_reads_a_frame(tmp_path):
    assert abi.HEADER_PATH.read_text() == abi.c_header(), "regenerate csrc/include/pie_bridge.h with abi.c_header()"
    frame = tmp_path / "frame.bin"
    frame.write_bytes(abi.pack_forward_request(_req()))
    src = tmp_path / "read.c"
    src.write_text('''
#include <stdio.h>
#include <stdlib.h>
#include "pie_bridge.h"
int main(int argc, char** argv) {
    FILE* f = fopen(argv[1], "rb"); static char buf[1 << 16]; size_t n = fread(buf, 1, sizeof buf, f); fclose(f);
    const PieFrameHeader* h = (const PieFrameHeader*)buf;
    if (h->frame_bytes != n || h->schema_hash64 != PIE_BRIDGE_SCHEMA_HASH64) return 2;
    const PieSection* s = pie_frame_section(buf, PIE_FORWARD_REQUEST_TOKENS);
    const int32_t* t = (const int32_t*)pie_section_data(buf, s);
    const PieSection* c = pie_frame_section(buf, PIE_FORWARD_REQUEST_CONTEXT_IDS);
    const uint64_t* ids = (const uint64_t*)pie_section_data(buf, c);
    printf("%d %llu %d %d %llu\\n", (int)h->kind, (unsigned long long)s->count, t[0], t[3], (unsigned long long)ids[1]);
    return pie_frame_section(buf, 9999) ? 3 : 0;
}''')
    exe = tmp_path / "read"
    subprocess.run(["gcc", "-Wall", "-Werror", "-I", str(abi.HEADER_PATH.parent), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe), str(frame)], check=True, capture_output=True, text=True).stdout.split()
    assert out == ["1", "4", "5", "8", str(2 ** 40)]


def _ring_reader(name, q):
    from pie_b200.parallel.comm import KIND_BATCH, KIND_COPY, StepRing
    ring = StepRing(name, 2, 1, cap=1 << 16, create=False)
    kind, payload, _ = ring.receive(timeout=30)
    req = abi.unpack_forward_request(payload.tobytes())
    ring.ack()
    kind2, payload2, _ = ring.receive(timeout=30)
    cp = abi.unpack_copy_request(payload2.tobytes())
    ring.ack()
    ring.close()
    q.put((kind == KIND_BATCH, req.tokens.tolist(), req.logit_masks, req.slot_samplers[0].seed,
           kind2 == KIND_COPY, cp.dsts.tolist()))


def test_frames_cross_the_shared_memory_ring():
    """The control ring of tensor parallelism carries wire frames between real processes."""
    import multiprocessing as mp
    import os
    from pie_b200.parallel.comm import KIND_BATCH, KIND_COPY, StepRing
    name = f"pie_b200_test_abi_{os.getpid()}"
    ring = StepRing(name, 2, 0, cap=1 << 16, create=True)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_ring_reader, args=(name, q))
    p.start()
    try:
        ring.publish(KIND_BATCH, np.frombuffer(abi.pack_forward_request(_req()), dtype=np.uint8))
        ring.publish(KIND_COPY, np.frombuffer(abi.pack_copy_request(
            CopyRequest(CopyDir(0), np.asarray([1], np.int32), np.asarray([9], np.int32))), dtype=np.uint8))
        got = q.get(timeout=60)
    finally:
        p.join(timeout=10)
        ring.close(unlink=True)
    assert got == (True, [5, 6, 7, 8], [None, [3, 5, 100]], 1234567890123, True, [9])
