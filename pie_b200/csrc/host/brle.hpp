// Binary run-length encoding of boolean vectors: a list of run lengths, alternating False,
// True, False ... starting with a (possibly empty) run of False. Native implementation of
// pie_b200/runtime/brle.py. Same encoding as the reference's driver/bridge/src/brle.rs:1-36.
#pragma once
#include <algorithm>
#include <cstdint>
#include <vector>

namespace pie_host {

using Brle = std::vector<uint32_t>;

inline Brle brle_encode(const uint8_t* bits, size_t n) {
    Brle out;
    if (n == 0) return out;
    if (bits[0]) out.push_back(0);
    size_t run = 1;
    for (size_t i = 1; i < n; ++i) {
        if ((bits[i] != 0) == (bits[i - 1] != 0)) {
            ++run;
        } else {
            out.push_back((uint32_t)run);
            run = 1;
        }
    }
    out.push_back((uint32_t)run);
    return out;
}

inline void brle_decode(const Brle& runs, uint8_t* out, size_t n, bool tail) {
    std::fill(out, out + n, tail ? 1 : 0);
    size_t pos = 0;
    for (size_t i = 0; i < runs.size() && pos < n; ++i) {
        const size_t end = std::min(n, pos + (size_t)runs[i]);
        if (i & 1) std::fill(out + pos, out + end, 1);
        else std::fill(out + pos, out + end, 0);
        pos = end;
    }
}

inline uint64_t brle_length(const Brle& r) {
    uint64_t s = 0;
    for (uint32_t x : r) s += x;
    return s;
}

inline uint64_t brle_count_true(const Brle& r) {
    uint64_t s = 0;
    for (size_t i = 1; i < r.size(); i += 2) s += r[i];
    return s;
}

// Streaming AND of two encodings without expanding them.
inline Brle brle_and(const Brle& a, const Brle& b) {
    Brle out;
    const uint64_t n = std::max(brle_length(a), brle_length(b));
    size_t ia = 0, ib = 0;
    uint64_t ra = ia < a.size() ? a[0] : n, rb = ib < b.size() ? b[0] : n;
    bool cur = false;
    uint64_t run = 0, pos = 0;
    auto value = [](size_t i, size_t size) { return i < size ? (i & 1) != 0 : false; };
    while (pos < n) {
        while (ra == 0 && ia < a.size()) { ++ia; ra = ia < a.size() ? a[ia] : n - pos; }
        while (rb == 0 && ib < b.size()) { ++ib; rb = ib < b.size() ? b[ib] : n - pos; }
        if (ra == 0) ra = n - pos;
        if (rb == 0) rb = n - pos;
        const uint64_t step = std::min({ra, rb, n - pos});
        const bool v = value(ia, a.size()) && value(ib, b.size());
        if (v == cur) {
            run += step;
        } else {
            out.push_back((uint32_t)run);
            cur = v;
            run = step;
        }
        ra -= step;
        rb -= step;
        pos += step;
    }
    out.push_back((uint32_t)run);
    return out;
}

// Packed bitmask (bit i of the vector at word i/32, bit i%32) of one encoding.
inline void brle_to_bitmask(const Brle& runs, uint32_t* words, size_t nbits, bool tail) {
    const size_t nw = (nbits + 31) / 32;
    std::fill(words, words + nw, 0u);
    auto set_range = [&](size_t a, size_t b) {
        for (size_t i = a; i < b;) {
            const size_t w = i >> 5, off = i & 31;
            const size_t take = std::min<size_t>(32 - off, b - i);
            const uint32_t m = take == 32 ? 0xffffffffu : (((1u << take) - 1u) << off);
            words[w] |= m;
            i += take;
        }
    };
    size_t pos = 0;
    for (size_t i = 0; i < runs.size() && pos < nbits; ++i) {
        const size_t end = std::min(nbits, pos + (size_t)runs[i]);
        if (i & 1) set_range(pos, end);
        pos = end;
    }
    if (tail && pos < nbits) set_range(pos, nbits);
}

// Pages whose positions are masked out in every row (page-trim candidates).
inline std::vector<uint8_t> brle_droppable_pages(const std::vector<Brle>& rows, int page_size, int num_pages) {
    std::vector<uint8_t> visible((size_t)num_pages, 0);
    for (const Brle& r : rows) {
        uint64_t pos = 0;
        for (size_t i = 0; i < r.size(); ++i) {
            const uint64_t end = pos + r[i];
            if ((i & 1) && r[i]) {
                const uint64_t p0 = pos / page_size, p1 = std::min<uint64_t>(num_pages, (end + page_size - 1) / page_size);
                for (uint64_t p = p0; p < p1; ++p) visible[p] = 1;
            }
            pos = end;
        }
    }
    std::vector<uint8_t> out((size_t)num_pages);
    for (int p = 0; p < num_pages; ++p) out[p] = !visible[p];
    return out;
}

}  // namespace pie_host
