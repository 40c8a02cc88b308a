"""Runtime <-> driver contract: plain structs in structure-of-arrays / CSR form.

Runtime and driver share one address space, so a request is a set of numpy arrays handed
over by reference: no serialisation step. Content-wise the structs carry what the
reference's wire schema carries (driver/bridge/src/schema.rs:83-286 ForwardRequest /
ForwardResponse, :196-233 Sampler, :293-353 Copy/Adapter requests;
driver/bridge/src/capabilities.rs:17-78 for the capability handshake).
"""
from __future__ import annotations

import enum
import json
from dataclasses import dataclass, field, asdict
from typing import List, Optional, Sequence

import numpy as np


class SamplerKind(enum.IntEnum):
    MULTINOMIAL = 0   # (temperature, seed)
    TOP_K = 1         # (temperature, k)
    TOP_P = 2         # (temperature, p)
    MIN_P = 3         # (temperature, p)
    TOP_K_TOP_P = 4   # (temperature, k, p)
    EMBEDDING = 5
    DIST = 6          # (temperature, k) -> top-k ids + probabilities
    RAW_LOGITS = 7
    LOGPROB = 8       # (token)
    LOGPROBS = 9      # (tokens...)
    ENTROPY = 10


TOKEN_SAMPLERS = {SamplerKind.MULTINOMIAL, SamplerKind.TOP_K, SamplerKind.TOP_P, SamplerKind.MIN_P,
                  SamplerKind.TOP_K_TOP_P}


@dataclass
class SamplerSpec:
    kind: SamplerKind = SamplerKind.MULTINOMIAL
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0                    # 0 = the driver draws a fresh seed for this fire
    labels: Sequence[int] = ()       # LOGPROB / LOGPROBS candidates
    seed_final: bool = False         # the seed is already the per-draw seed (set by the cohort's CPU path)

    @property
    def is_token(self) -> bool:
        return self.kind in TOKEN_SAMPLERS

    @staticmethod
    def greedy() -> "SamplerSpec":
        return SamplerSpec(SamplerKind.MULTINOMIAL, temperature=0.0)


@dataclass
class SlotOutput:
    """One typed result per sampler slot, in attach order."""
    kind: str                         # token | distribution | logits | logprobs | entropy | embedding
    token: int = 0
    ids: Optional[list] = None
    probs: Optional[list] = None
    logits: Optional[bytes] = None
    logprobs: Optional[list] = None
    entropy: float = 0.0


@dataclass
class ForwardRequest:
    """A batch of R requests with N input tokens in total."""
    tokens: np.ndarray                 # int32 [N]
    positions: np.ndarray              # int32 [N]
    qo_indptr: np.ndarray              # int32 [R+1]
    kv_page_indices: np.ndarray        # int32 [sum pages]  active prefix of each request's pages
    kv_page_indptr: np.ndarray         # int32 [R+1]
    kv_last_page_lens: np.ndarray      # int32 [R]   tokens in the last page AFTER this pass
    # attention masks: BRLE per input token row for requests with has_user_mask, else causal
    has_user_mask: np.ndarray = None   # bool [R]
    mask_runs: Optional[list] = None   # list over token rows (only rows of masked requests) of BRLE lists
    mask_row_indptr: Optional[np.ndarray] = None  # int32 [R+1] rows of mask_runs per request
    # constrained decoding: one BRLE over the vocabulary per request (None = no mask)
    logit_masks: Optional[list] = None
    # sampling slots
    slot_req: np.ndarray = None        # int32 [S] request of each slot
    slot_row: np.ndarray = None        # int32 [S] token row (global index into tokens) of each slot
    slot_samplers: List[SamplerSpec] = field(default_factory=list)
    # speculative drafts already spliced into tokens: number of draft tokens per request
    # models with recurrent (linear-attention) layers: the state slot of every request, and which slots
    # must start from zero in this fire (first pass of a context, or a replay after its state was lost)
    rs_slots: Optional[np.ndarray] = None     # int32 [R]
    rs_reset: Optional[np.ndarray] = None     # int32 [R]
    spec_counts: Optional[np.ndarray] = None
    # media side channel: spans of token rows whose embeddings come from an encoded image / video / audio clip that
    # the driver holds under `media_slot` (see `put_media`): rows media_dst[i] .. +media_count[i] of this batch take
    # rows media_src[i] .. of that clip's encoder output instead of the token embedding
    media_slot: Optional[np.ndarray] = None        # int32 [M]
    media_src: Optional[np.ndarray] = None         # int32 [M]
    media_dst: Optional[np.ndarray] = None         # int32 [M]
    media_count: Optional[np.ndarray] = None       # int32 [M]
    context_ids: Optional[np.ndarray] = None       # uint64 [R]
    adapter_ids: Optional[np.ndarray] = None       # int64 [R], -1 = none
    single_token_mode: bool = False                # every request has exactly one input token
    trimmed_pages: int = 0                         # pages dropped by the runtime's page trim (statistics)

    @property
    def num_requests(self) -> int:
        return len(self.qo_indptr) - 1

    @property
    def num_tokens(self) -> int:
        return len(self.tokens)


# Placeholder tokens of media rows: a context's lineage stores MEDIA_TOKEN_BASE + slot * MEDIA_ROWS + row for row
# `row` of the clip in media slot `slot`. They hash and replay like any token (the same clip gives the same
# placeholders, so its pages are shared); the request builder turns them into media spans and sends token 0.
MEDIA_TOKEN_BASE = 1 << 30
MEDIA_ROWS = 1 << 16
MEDIA_SLOTS = (1 << 30) // MEDIA_ROWS


def media_tokens(slot: int, count: int, start: int = 0) -> List[int]:
    if not 0 <= slot < MEDIA_SLOTS or start + count > MEDIA_ROWS:
        raise ValueError(f"media slot {slot} / rows {start}+{count} outside the placeholder range")
    base = MEDIA_TOKEN_BASE + slot * MEDIA_ROWS + start
    return list(range(base, base + count))


def split_media_spans(tokens: np.ndarray):
    """(tokens with placeholders replaced by 0, slot, src, dst, count) - the four arrays are None when no token
    is a media placeholder. Consecutive rows of one clip form one span."""
    tokens = np.asarray(tokens, dtype=np.int32)
    if tokens.size == 0 or int(tokens.max()) < MEDIA_TOKEN_BASE:
        return tokens, None, None, None, None
    dst = np.flatnonzero(tokens >= MEDIA_TOKEN_BASE).astype(np.int32)
    code = tokens[dst] - MEDIA_TOKEN_BASE
    slot, row = code // MEDIA_ROWS, code % MEDIA_ROWS
    brk = np.flatnonzero((np.diff(dst) != 1) | (np.diff(slot) != 0) | (np.diff(row) != 1)) + 1
    starts = np.concatenate([[0], brk])
    counts = np.diff(np.concatenate([starts, [len(dst)]]))
    out = tokens.copy()
    out[dst] = 0
    return out, slot[starts].astype(np.int32), row[starts].astype(np.int32), dst[starts], counts.astype(np.int32)


@dataclass
class ForwardResponse:
    slots: List[SlotOutput]
    # pure token fast path: tokens[i] is the sampled token of slot i when every slot is a token sampler
    tokens: Optional[np.ndarray] = None
    # phase timings in microseconds (the reference returns 6 probe fields per response)
    t_build_us: float = 0.0
    t_h2d_us: float = 0.0
    t_forward_us: float = 0.0
    t_sample_us: float = 0.0
    t_d2h_us: float = 0.0
    t_total_us: float = 0.0
    # drafts accepted per request (int32 [R]) when the request carried `spec_counts`: the driver verifies
    # each draft against the token it sampled at the previous row
    spec_accepted: Optional[np.ndarray] = None


def verify_drafts(req: "ForwardRequest", slot_tokens: dict) -> np.ndarray:
    """Accepted draft count per request. The last `spec_counts[r]` input tokens of request r are drafts;
    draft j stands while the token sampled at the row before it (`slot_tokens`: row -> sampled token)
    equals it. Counterpart of the driver-side speculation expansion of the reference
    (driver/cuda/src/executor/spec_expand.cpp)."""
    qo = np.asarray(req.qo_indptr)
    out = np.zeros(len(qo) - 1, np.int32)
    for r, k in enumerate(np.asarray(req.spec_counts)):
        end = int(qo[r + 1])
        for j in range(int(k)):
            row = end - int(k) + j
            if slot_tokens.get(row - 1) != int(req.tokens[row]):
                break
            out[r] += 1
    return out


class CopyDir(enum.IntEnum):
    D2D = 0
    D2H = 1
    H2D = 2
    H2H = 3


@dataclass
class CopyRequest:
    direction: CopyDir
    srcs: np.ndarray   # int32 page ids (device pool for D2*, host pool for H2*)
    dsts: np.ndarray


@dataclass
class Capabilities:
    """What a driver advertises at start-up; the runtime batches against these limits."""
    total_pages: int = 0
    kv_page_size: int = 16
    swap_pool_size: int = 0
    max_forward_tokens: int = 8192
    max_forward_requests: int = 512
    max_page_refs: int = 1 << 20
    max_logit_rows: int = 1024
    max_prob_rows: int = 1024
    max_sampler_rows: int = 1024
    max_logprob_labels: int = 4096
    max_custom_mask_bytes: int = 1 << 26
    arch_name: str = ""
    vocab_size: int = 0
    max_model_len: int = 0
    activation_dtype: str = "bfloat16"
    tp_size: int = 1
    system_speculation: bool = False
    rs_cache_slots: int = 0
    cohort_decode: bool = True      # False: no array-form decode step (`decode_async`); the runtime steps per request
    media: tuple = ()               # media kinds the driver can encode ("image", "video", "audio"); empty for text-only models
    media_spec: dict = field(default_factory=dict)   # what the host's preprocessing must produce for the model's vision tower:
                                    # {"style": "qwen", "patch", "merge", "temporal"} or {"style": "siglip", "image_size", "patch", "pool"}

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @staticmethod
    def from_json(s: str) -> "Capabilities":
        d = json.loads(s)
        d["media"] = tuple(d.get("media") or ())
        return Capabilities(**d)


_SEED_MIX = np.int64(0x9E3779B97F4A7C15 - (1 << 64))


def position_seed(seed, position):
    """Per-draw sampler seed of a request that fixed its own seed: the user's seed mixed with the
    position of the input token whose row is sampled, so that every decode step draws fresh noise
    and both scheduler paths (per-request fires and the array-stepped cohort) produce the same
    stream. Works on scalars and numpy arrays; never returns 0 (0 means "pick a seed per fire")."""
    with np.errstate(over="ignore"):
        out = (np.asarray(seed, dtype=np.int64) * _SEED_MIX) ^ (np.asarray(position, dtype=np.int64) * np.int64(0x632BE5AB))
    return np.where(out == 0, 1, out)
