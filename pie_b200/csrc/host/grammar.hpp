// Constrained decoding engine: a byte-level nondeterministic pushdown matcher over a context-free
// grammar plus a token-trie walk that turns the current parser state into a vocabulary mask.
//
// Grammar IR (built by the Python front ends from EBNF / regex / JSON schema): rules[r] is a list
// of alternatives, an alternative a list of symbols; a symbol is a byte class (256-bit set) or a
// reference to a rule. Repetition and grouping are desugared into extra rules by the front end.
// Matcher state = a set of parse stacks (frames: rule, alternative, position), each closed so
// that its top frame points at a byte class (or the stack is empty = accepting).
// next_token_mask() walks the trie of token byte strings depth first, advancing the state set
// byte by byte and pruning dead branches, so the cost follows the live part of the vocabulary.
//
// Counterpart of the reference's structured decoding engine (runtime/src/inference/structured/
// {compiled_grammar,matcher,stack_parser,bitmask}.rs); the approach (token trie x stack parser)
// is the same family, the code is new.
#pragma once
#include <algorithm>
#include <array>
#include <cstdint>
#include <list>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace pie_host {

struct GSymbol {
    bool is_rule = false;
    int rule = -1;
    std::array<uint64_t, 4> cls{};   // byte class when !is_rule
    bool has(unsigned char b) const { return (cls[b >> 6] >> (b & 63)) & 1ull; }
};

// Token masks by matcher state, shared by every matcher of one grammar (the state of a pushdown
// matcher recurs constantly: every character inside a JSON string, every digit of a number, every
// item of an array leads back to a state seen before). Key: an order-independent 128-bit digest of
// the set of parse stacks plus the trie the mask was computed against; value: the allowed-token
// bytes. Least-recently-used entries go first. Counterpart of the adaptive token-mask cache of the
// reference's compiled grammar (runtime/src/inference/structured/compiled_grammar.rs:21-50).
struct MaskCache {
    struct Key {
        uint64_t a, b;
        const void* trie;
        bool operator==(const Key& o) const { return a == o.a && b == o.b && trie == o.trie; }
    };
    struct KeyHash {
        size_t operator()(const Key& k) const { return (size_t)(k.a ^ (k.b * 0x9E3779B97F4A7C15ull) ^ (uintptr_t)k.trie); }
    };
    using Entry = std::pair<Key, std::shared_ptr<const std::vector<uint8_t>>>;
    size_t capacity = 512;
    mutable std::mutex mu;
    mutable std::list<Entry> lru;
    mutable std::unordered_map<Key, std::list<Entry>::iterator, KeyHash> index;
    mutable uint64_t hits = 0, misses = 0;

    std::shared_ptr<const std::vector<uint8_t>> find(const Key& k) const {
        std::lock_guard<std::mutex> lock(mu);
        auto it = index.find(k);
        if (it == index.end()) {
            ++misses;
            return nullptr;
        }
        ++hits;
        lru.splice(lru.begin(), lru, it->second);
        return it->second->second;
    }
    void put(const Key& k, std::shared_ptr<const std::vector<uint8_t>> v) const {
        std::lock_guard<std::mutex> lock(mu);
        if (index.count(k)) return;
        lru.emplace_front(k, std::move(v));
        index[k] = lru.begin();
        while (lru.size() > capacity) {
            index.erase(lru.back().first);
            lru.pop_back();
        }
    }
};

struct GFrame {
    int rule, alt, pos;
    bool operator==(const GFrame& o) const { return rule == o.rule && alt == o.alt && pos == o.pos; }
};
using GStack = std::vector<GFrame>;

// Lazily built automaton over matcher states: a state set gets a number the first time it is seen,
// and the successor of (state, byte) is computed once. The token-trie walk of a mask then moves
// through table look-ups wherever the grammar has been before. Bounded: past `max_states` the walk
// falls back to computing successors directly.
struct StateTable {
    static constexpr int kUnknown = -2, kDead = -1;
    size_t max_states = 16384;
    std::mutex mu;
    std::unordered_map<uint64_t, std::vector<int>> by_hash;          // digest -> candidate ids
    std::vector<std::shared_ptr<const std::vector<GStack>>> sets;
    std::vector<std::array<int, 256>> trans;
};

struct Grammar {
    std::vector<std::vector<std::vector<GSymbol>>> rules;   // rule -> alternatives -> symbols
    int root = 0;
    MaskCache mask_cache;
    mutable StateTable table;
};

inline uint64_t gstack_hash(const GStack& s) {
    uint64_t h = 0x9E3779B97F4A7C15ull ^ s.size();
    for (const GFrame& f : s) {
        uint64_t x = ((uint64_t)(uint32_t)f.rule << 40) ^ ((uint64_t)(uint32_t)f.alt << 20) ^ (uint32_t)f.pos;
        h ^= x + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    }
    return h;
}

struct TokenTrie {
    struct Node {
        int child[256];
        std::vector<int> tokens;   // token ids ending here
        Node() { std::fill(child, child + 256, -1); }
    };
    std::vector<Node> nodes;
    int vocab = 0;
    TokenTrie() { nodes.emplace_back(); }
    void insert(int id, const std::string& bytes) {
        if (bytes.empty()) return;
        int n = 0;
        for (unsigned char c : bytes) {
            if (nodes[n].child[c] < 0) {
                nodes[n].child[c] = (int)nodes.size();
                nodes.emplace_back();
            }
            n = nodes[n].child[c];
        }
        nodes[n].tokens.push_back(id);
        vocab = std::max(vocab, id + 1);
    }
};

class GrammarMatcher {
public:
    static constexpr size_t kMaxStates = 8192;
    static constexpr size_t kMaxDepth = 512;

    GrammarMatcher(const Grammar* g, const TokenTrie* trie) : g_(g), trie_(trie) { reset(); }

    void reset() {
        history_.clear();
        states_.clear();
        std::vector<GStack> init;
        for (int a = 0; a < (int)g_->rules[g_->root].size(); ++a) init.push_back(GStack{GFrame{g_->root, a, 0}});
        closure(init, states_);
    }

    // Advance by the bytes of one token; false (state unchanged) when the grammar rejects them.
    bool accept_bytes(const std::string& bytes) {
        std::vector<GStack> cur = states_;
        for (unsigned char c : bytes) {
            std::vector<GStack> nxt;
            step(cur, c, nxt);
            if (nxt.empty()) return false;
            cur.swap(nxt);
        }
        history_.push_back(states_);
        if (history_.size() > 64) history_.erase(history_.begin());
        states_.swap(cur);
        return true;
    }

    // Undo the last n accepted tokens (bounded history).
    bool rollback(int n) {
        if (n <= 0) return true;
        if ((size_t)n > history_.size()) return false;
        states_ = history_[history_.size() - n];
        history_.resize(history_.size() - n);
        return true;
    }

    bool can_terminate() const {
        for (const GStack& s : states_)
            if (s.empty()) return true;
        return false;
    }
    // Terminated = the only way forward is to stop.
    bool is_terminated() const {
        if (states_.empty()) return true;
        for (const GStack& s : states_)
            if (!s.empty()) return false;
        return true;
    }
    size_t num_states() const { return states_.size(); }

    // allowed[id] = 1 for every token whose bytes the grammar accepts from the current state.
    // Served from the grammar's mask cache when this state set was seen before (by any matcher).
    void next_token_mask(std::vector<uint8_t>& allowed) const {
        const MaskCache::Key key = state_key();
        if (auto hit = g_->mask_cache.find(key)) {
            allowed = *hit;
            return;
        }
        allowed.assign((size_t)trie_->vocab, 0);
        const int id = intern(states_);
        if (id >= 0) walk_table(0, id, allowed);
        else walk(0, states_, allowed);
        g_->mask_cache.put(key, std::make_shared<const std::vector<uint8_t>>(allowed));
    }

    // Digest of the state set, independent of the order the stacks were produced in.
    MaskCache::Key state_key() const {
        uint64_t a = 0x243F6A8885A308D3ull ^ states_.size(), b = 0;
        for (const GStack& s : states_) {
            const uint64_t h = gstack_hash(s);
            a += h * 0xD6E8FEB86659FD93ull;                       // commutative combination: order does not matter
            b ^= (h ^ (h >> 29)) * 0xBF58476D1CE4E5B9ull + 0x94D049BB133111EBull;
        }
        return MaskCache::Key{a, b, (const void*)trie_};
    }

private:
    const Grammar* g_;
    const TokenTrie* trie_;
    std::vector<GStack> states_;
    std::vector<std::vector<GStack>> history_;

    const GSymbol* top_symbol(const GStack& s) const {
        const GFrame& f = s.back();
        const auto& alt = g_->rules[f.rule][f.alt];
        return f.pos < (int)alt.size() ? &alt[f.pos] : nullptr;
    }

    // Expand rule references / pop finished frames until every stack is empty or at a byte class.
    void closure(std::vector<GStack>& work, std::vector<GStack>& out) const {
        std::unordered_set<uint64_t> seen;
        while (!work.empty() && out.size() < kMaxStates) {
            GStack s = std::move(work.back());
            work.pop_back();
            if (!seen.insert(gstack_hash(s)).second) continue;
            if (s.empty()) {
                out.push_back(std::move(s));
                continue;
            }
            const GSymbol* sym = top_symbol(s);
            if (sym == nullptr) {           // alternative finished: return to the caller frame
                s.pop_back();
                if (!s.empty()) s.back().pos += 1;
                work.push_back(std::move(s));
            } else if (sym->is_rule) {
                // A reference that is the last symbol of its alternative is a tail call: the frame is
                // replaced, not stacked (when the callee finishes, the frame below advances, which is
                // what the finished caller would have done). Repetition desugars to right recursion, so
                // this keeps the stack - and with it the matcher state - the same from one iteration to
                // the next: long strings do not deepen the stack and their states recur in the mask cache.
                const GFrame top = s.back();
                const bool tail = top.pos + 1 == (int)g_->rules[top.rule][top.alt].size();
                if (!tail && s.size() >= kMaxDepth) continue;
                for (int a = 0; a < (int)g_->rules[sym->rule].size(); ++a) {
                    GStack t = s;
                    if (tail) t.back() = GFrame{sym->rule, a, 0};
                    else t.push_back(GFrame{sym->rule, a, 0});
                    work.push_back(std::move(t));
                }
            } else {
                out.push_back(std::move(s));
            }
        }
    }

    void step(const std::vector<GStack>& cur, unsigned char c, std::vector<GStack>& out) const {
        std::vector<GStack> work;
        for (const GStack& s : cur) {
            if (s.empty()) continue;
            const GSymbol* sym = top_symbol(s);
            if (sym && !sym->is_rule && sym->has(c)) {
                GStack t = s;
                t.back().pos += 1;
                work.push_back(std::move(t));
            }
        }
        closure(work, out);
    }

    static uint64_t set_digest(const std::vector<GStack>& st) {
        uint64_t a = 0x243F6A8885A308D3ull ^ st.size();
        for (const GStack& s : st) a += gstack_hash(s) * 0xD6E8FEB86659FD93ull;
        return a;
    }
    static bool same_set(const std::vector<GStack>& x, const std::vector<GStack>& y) {
        if (x.size() != y.size()) return false;
        for (const GStack& s : x)
            if (std::find(y.begin(), y.end(), s) == y.end()) return false;
        return true;
    }
    // Number of a state set in the grammar's table (-1 when the table is full).
    int intern(const std::vector<GStack>& st) const {
        StateTable& t = g_->table;
        const uint64_t d = set_digest(st);
        std::lock_guard<std::mutex> lock(t.mu);
        auto& ids = t.by_hash[d];
        for (int id : ids)
            if (same_set(*t.sets[id], st)) return id;
        if (t.sets.size() >= t.max_states) return -1;
        const int id = (int)t.sets.size();
        t.sets.push_back(std::make_shared<const std::vector<GStack>>(st));
        std::array<int, 256> row;
        row.fill(StateTable::kUnknown);
        t.trans.push_back(row);
        ids.push_back(id);
        return id;
    }
    // Successor of table state `id` on byte c: kDead, a table id, or kUnknown when the table is full
    // (then *overflow holds the successor set).
    int next_state(int id, unsigned char c, std::vector<GStack>* overflow) const {
        StateTable& t = g_->table;
        std::shared_ptr<const std::vector<GStack>> cur;
        {
            std::lock_guard<std::mutex> lock(t.mu);
            const int known = t.trans[id][c];
            if (known != StateTable::kUnknown) return known;
            cur = t.sets[id];
        }
        std::vector<GStack> nxt;
        step(*cur, c, nxt);
        int to = StateTable::kDead;
        if (!nxt.empty()) {
            to = intern(nxt);
            if (to < 0) {
                *overflow = std::move(nxt);
                return StateTable::kUnknown;
            }
        }
        std::lock_guard<std::mutex> lock(t.mu);
        t.trans[id][c] = to;
        return to;
    }
    void walk_table(int node, int id, std::vector<uint8_t>& allowed) const {
        const TokenTrie::Node& n = trie_->nodes[node];
        for (int tok : n.tokens) allowed[tok] = 1;
        for (int c = 0; c < 256; ++c) {
            if (n.child[c] < 0) continue;
            std::vector<GStack> overflow;
            const int to = next_state(id, (unsigned char)c, &overflow);
            if (to >= 0) walk_table(n.child[c], to, allowed);
            else if (to == StateTable::kUnknown) walk(n.child[c], overflow, allowed);
        }
    }

    void walk(int node, const std::vector<GStack>& st, std::vector<uint8_t>& allowed) const {
        const TokenTrie::Node& n = trie_->nodes[node];
        for (int id : n.tokens) allowed[id] = 1;
        // bytes any live stack can take next
        std::array<uint64_t, 4> live{};
        for (const GStack& s : st) {
            if (s.empty()) continue;
            const GSymbol* sym = top_symbol(s);
            if (sym && !sym->is_rule)
                for (int w = 0; w < 4; ++w) live[w] |= sym->cls[w];
        }
        for (int c = 0; c < 256; ++c) {
            if (n.child[c] < 0 || !((live[c >> 6] >> (c & 63)) & 1ull)) continue;
            std::vector<GStack> nxt;
            step(st, (unsigned char)c, nxt);
            if (!nxt.empty()) walk(n.child[c], nxt, allowed);
        }
    }
};

}  // namespace pie_host
