// Byte-pair-encoding merge engine. The vocabulary maps raw byte strings to ids; merges are
// ranked pairs of byte strings. A pre-tokenised piece (bytes) is encoded by starting from its
// single-byte tokens and repeatedly applying the lowest-ranked applicable merge. Pieces that are
// whole vocabulary entries short-circuit, and results are cached.
// Counterpart of the reference's own BPE (runtime/src/model/tokenizer/bpe.rs).
#pragma once
#include <cstdint>
#include <limits>
#include <string>
#include <unordered_map>
#include <vector>

namespace pie_host {

class BpeCore {
public:
    BpeCore(const std::vector<std::string>& vocab_bytes, const std::vector<int>& vocab_ids,
            const std::vector<std::pair<std::string, std::string>>& merges, int unk_id, bool byte_fallback)
        : unk_id_(unk_id), byte_fallback_(byte_fallback) {
        int max_id = -1;
        for (size_t i = 0; i < vocab_bytes.size(); ++i) {
            tok2id_[vocab_bytes[i]] = vocab_ids[i];
            if (vocab_ids[i] > max_id) max_id = vocab_ids[i];
        }
        id2tok_.assign(max_id + 1, std::string());
        for (size_t i = 0; i < vocab_bytes.size(); ++i) id2tok_[vocab_ids[i]] = vocab_bytes[i];
        for (int b = 0; b < 256; ++b) {
            auto it = tok2id_.find(std::string(1, (char)b));
            byte_id_[b] = it == tok2id_.end() ? -1 : it->second;
        }
        if (byte_fallback_) {
            static const char* hex = "0123456789ABCDEF";
            for (int b = 0; b < 256; ++b) {
                if (byte_id_[b] >= 0) continue;
                std::string name = "<0x";
                name += hex[b >> 4];
                name += hex[b & 15];
                name += ">";
                auto it = tok2id_.find(name);
                if (it != tok2id_.end()) byte_id_[b] = it->second;
            }
        }
        int rank = 0;
        for (auto& m : merges) {
            auto a = tok2id_.find(m.first), b = tok2id_.find(m.second), ab = tok2id_.find(m.first + m.second);
            if (a != tok2id_.end() && b != tok2id_.end() && ab != tok2id_.end()) {
                const uint64_t key = ((uint64_t)(uint32_t)a->second << 32) | (uint32_t)b->second;
                if (!ranks_.count(key)) ranks_[key] = {rank, ab->second};
            }
            ++rank;
        }
    }

    std::vector<int> encode_piece(const std::string& piece) {
        std::vector<int> out;
        if (piece.empty()) return out;
        auto whole = tok2id_.find(piece);
        if (whole != tok2id_.end()) {
            out.push_back(whole->second);
            return out;
        }
        auto hit = cache_.find(piece);
        if (hit != cache_.end()) return hit->second;
        // initial symbols: whole UTF-8 characters that are vocabulary entries (sentencepiece-style
        // vocabularies), single bytes otherwise (byte-level vocabularies, byte fallback)
        std::vector<int> ids;
        ids.reserve(piece.size());
        for (size_t i = 0; i < piece.size();) {
            const unsigned char c = (unsigned char)piece[i];
            size_t len = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1;
            if (i + len > piece.size()) len = 1;
            if (len > 1) {
                auto it = tok2id_.find(piece.substr(i, len));
                if (it != tok2id_.end()) {
                    ids.push_back(it->second);
                    i += len;
                    continue;
                }
                len = 1;
            }
            ids.push_back(byte_id_[c] >= 0 ? byte_id_[c] : unk_id_);
            i += 1;
        }
        while (ids.size() > 1) {
            int best_rank = std::numeric_limits<int>::max(), best_i = -1, best_id = -1;
            for (size_t i = 0; i + 1 < ids.size(); ++i) {
                const uint64_t key = ((uint64_t)(uint32_t)ids[i] << 32) | (uint32_t)ids[i + 1];
                auto it = ranks_.find(key);
                if (it != ranks_.end() && it->second.first < best_rank) {
                    best_rank = it->second.first;
                    best_i = (int)i;
                    best_id = it->second.second;
                }
            }
            if (best_i < 0) break;
            ids[best_i] = best_id;
            ids.erase(ids.begin() + best_i + 1);
        }
        if (cache_.size() < 200000) cache_[piece] = ids;
        return ids;
    }

    std::vector<int> encode_pieces(const std::vector<std::string>& pieces) {
        std::vector<int> out;
        for (auto& p : pieces) {
            auto ids = encode_piece(p);
            out.insert(out.end(), ids.begin(), ids.end());
        }
        return out;
    }

    std::string decode(const std::vector<int>& ids) const {
        std::string out;
        for (int id : ids)
            if (id >= 0 && id < (int)id2tok_.size()) out += id2tok_[id];
        return out;
    }

    int vocab_size() const { return (int)id2tok_.size(); }
    const std::string& token_bytes(int id) const { return id2tok_.at(id); }

private:
    int unk_id_;
    bool byte_fallback_;
    int byte_id_[256];
    std::unordered_map<std::string, int> tok2id_;
    std::vector<std::string> id2tok_;
    std::unordered_map<uint64_t, std::pair<int, int>> ranks_;
    std::unordered_map<std::string, std::vector<int>> cache_;
};

}  // namespace pie_host
