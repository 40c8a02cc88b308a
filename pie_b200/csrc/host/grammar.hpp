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
#include <string>
#include <unordered_set>
#include <vector>

namespace pie_host {

struct GSymbol {
    bool is_rule = false;
    int rule = -1;
    std::array<uint64_t, 4> cls{};   // byte class when !is_rule
    bool has(unsigned char b) const { return (cls[b >> 6] >> (b & 63)) & 1ull; }
};

struct Grammar {
    std::vector<std::vector<std::vector<GSymbol>>> rules;   // rule -> alternatives -> symbols
    int root = 0;
};

struct GFrame {
    int rule, alt, pos;
    bool operator==(const GFrame& o) const { return rule == o.rule && alt == o.alt && pos == o.pos; }
};
using GStack = std::vector<GFrame>;

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
    void next_token_mask(std::vector<uint8_t>& allowed) const {
        allowed.assign((size_t)trie_->vocab, 0);
        walk(0, states_, allowed);
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
                if (s.size() >= kMaxDepth) continue;
                for (int a = 0; a < (int)g_->rules[sym->rule].size(); ++a) {
                    GStack t = s;
                    t.push_back(GFrame{sym->rule, a, 0});
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
