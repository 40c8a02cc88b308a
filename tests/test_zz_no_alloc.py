"""The allocation-free decode-attention entry point (`pie_paged_decode_attn_noalloc`).

It serves callers that cannot allocate device memory once serving has started: the KV pool owns
nearly all of the GPU, and a cudaMalloc at that point may fail and always stalls the device.
The test calls the exported C symbol directly (ctypes, no wrapper) twice in a row with different
inputs and checks each result against the ordinary entry point, which takes caller-owned scratch.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = -1001
SCRATCH_FLOATS = 4 * 1024 * 1024


def _setup(seed, kv_lens, hq=32, hkv=8, d=128, page=16):
    from pie_b200 import ops
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    r = len(kv_lens)
    npages = [-(-int(k) // page) for k in kv_lens]
    total = sum(npages) + 3
    kv = (torch.randn(total, 2, hkv, page, d, generator=g, device=dev)).to(torch.bfloat16)
    pages = torch.randperm(total, generator=torch.Generator().manual_seed(seed))[: sum(npages)].numpy().astype(np.int32)
    indptr = np.zeros(r + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(npages)
    q = torch.randn(r, hq, d, generator=g, device=dev).to(torch.bfloat16)
    item_req, st, en, iptr = ops.plan_decode_items(np.asarray(kv_lens), hkv, target_ctas=64, min_chunk=256)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    return dict(q=q, kv=kv, pages=t(pages), indptr=t(indptr), item_req=t(item_req), item_start=t(st),
                item_end=t(en), iptr=t(iptr), n_items=torch.tensor([len(item_req)], dtype=torch.int32, device=dev),
                max_items=len(item_req) + 2, r=r, hq=hq, hkv=hkv, d=d, page=page)


def _call_both(lib, s):
    from pie_b200 import ops
    p = lambda x: C.c_void_p(x.data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = C.c_float(1.0 / math.sqrt(s["d"]))
    out_ref = torch.zeros_like(s["q"])
    out_new = torch.zeros_like(s["q"])
    scratch = torch.empty(ops.decode_scratch_floats(s["max_items"], s["hq"], s["d"]), device="cuda")
    rc = lib.pie_paged_decode_attn(p(s["q"]), p(s["kv"]), p(s["pages"]), p(s["indptr"]), p(s["item_req"]),
                                   p(s["item_start"]), p(s["item_end"]), p(s["iptr"]), p(s["n_items"]), p(out_ref),
                                   p(scratch), s["max_items"], s["r"], s["hq"], s["hkv"], s["d"], s["page"], scale,
                                   64, 1, stream)
    assert rc == 0
    fn = lib.pie_paged_decode_attn_noalloc
    fn.restype = C.c_int
    rc = fn(p(s["q"]), p(s["kv"]), p(s["pages"]), p(s["indptr"]), p(s["item_req"]), p(s["item_start"]),
            p(s["item_end"]), p(s["iptr"]), p(s["n_items"]), p(out_new), C.c_int(s["max_items"]), C.c_int(s["r"]),
            C.c_int(s["hq"]), C.c_int(s["hkv"]), C.c_int(s["d"]), C.c_int(s["page"]), scale, C.c_int(64), stream)
    assert rc == 0
    torch.cuda.synchronize()
    return out_ref, out_new


def test_noalloc_entry_point_matches_regular_entry_point_twice():
    from pie_b200.ops import _lib
    lib = _lib.load(required=True)
    for seed, kv_lens in ((1, [1, 17, 300, 1000, 2305, 64]), (2, [700, 5, 1500, 33, 2048, 256, 900])):
        s = _setup(seed, kv_lens)
        ref, new = _call_both(lib, s)
        err = (ref.float() - new.float()).abs()
        tol = 2e-2 + 2e-2 * ref.float().abs()
        assert bool((err <= tol).all()), f"seed {seed}: max err {err.max().item()}"
        assert float(new.float().abs().max()) > 0


def test_noalloc_rejects_oversized_requests():
    from pie_b200.ops import _lib
    lib = _lib.load(required=True)
    s = _setup(3, [64, 64])
    fn = lib.pie_paged_decode_attn_noalloc
    fn.restype = C.c_int
    p = lambda x: C.c_void_p(x.data_ptr())
    too_many = SCRATCH_FLOATS // (s["hq"] * (s["d"] + 1)) + 1
    out = torch.zeros_like(s["q"])
    rc = fn(p(s["q"]), p(s["kv"]), p(s["pages"]), p(s["indptr"]), p(s["item_req"]), p(s["item_start"]),
            p(s["item_end"]), p(s["iptr"]), p(s["n_items"]), p(out), C.c_int(too_many), C.c_int(s["r"]),
            C.c_int(s["hq"]), C.c_int(s["hkv"]), C.c_int(s["d"]), C.c_int(s["page"]), C.c_float(0.1), C.c_int(64),
            C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == TOO_LARGE
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0    # nothing was launched
