// Physical KV page pool and content-addressed store of committed pages (native implementation
// of pie_b200/runtime/pagestore.py, same API). Chained 64-bit page hashes key a flat map, which
// is equivalent to a radix trie over page chains; nodes carry path-inclusive reference counts.
// Behavioural counterpart of the reference's runtime/src/context/pagestore.rs:41-138 (pool with
// double-free detection), :152-602 (trie), :952-1006 (chained content hash).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <unordered_map>
#include <vector>

namespace pie_host {

class PagePool {
public:
    explicit PagePool(int num_pages) : num_pages_(num_pages), is_free_(num_pages, 1) {
        free_.reserve(num_pages);
        for (int p = num_pages - 1; p >= 0; --p) free_.push_back(p);
    }
    int num_pages() const { return num_pages_; }
    int free_count() const { return (int)free_.size(); }
    int used_count() const { return num_pages_ - (int)free_.size(); }
    int double_free_count() const { return double_free_; }
    // Returns false (and allocates nothing) when fewer than n pages are free.
    bool alloc(int n, std::vector<int>& out) {
        if (n > (int)free_.size()) return false;
        for (int i = 0; i < n; ++i) {
            const int p = free_.back();
            free_.pop_back();
            is_free_[p] = 0;
            out.push_back(p);
        }
        return true;
    }
    void free(const std::vector<int>& pages) {
        for (int p : pages) {
            if (p < 0 || p >= num_pages_) throw std::out_of_range("page id out of range");
            if (is_free_[p]) { ++double_free_; continue; }
            is_free_[p] = 1;
            free_.push_back(p);
        }
    }

private:
    int num_pages_;
    int double_free_ = 0;
    std::vector<int> free_;
    std::vector<uint8_t> is_free_;
};

// 64-bit mix (splitmix finaliser) chained over the page content.
inline uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

inline uint64_t page_hash(uint64_t prev, const uint32_t* tokens, const uint32_t* positions, size_t n,
                          const uint8_t* mask_key, size_t mask_len, uint64_t adapter_seed) {
    uint64_t h = mix64(prev ^ mix64(adapter_seed + 0x51ull) ^ (uint64_t)n);
    for (size_t i = 0; i < n; ++i) h = mix64(h ^ (((uint64_t)tokens[i] << 32) | positions[i]));
    for (size_t i = 0; i < mask_len; ++i) h = mix64(h ^ mask_key[i]);
    return h ? h : 1;
}

class PageStore {
public:
    explicit PageStore(int num_pages) : pool(num_pages) {}
    PagePool pool;

    struct Node {
        int page;
        uint64_t parent;
        int refcount;
        int children;
    };

    int lookup(uint64_t h) const {
        auto it = nodes_.find(h);
        return it == nodes_.end() ? -1 : it->second.page;
    }
    // Attach a filled page as node `h`; returns {page to use, deduplicated}.
    std::pair<int, bool> extend(uint64_t parent, uint64_t h, int page) {
        auto it = nodes_.find(h);
        if (it != nodes_.end()) {
            it->second.refcount += 1;
            return {it->second.page, true};
        }
        nodes_[h] = Node{page, parent, 1, 0};
        auto pit = nodes_.find(parent);
        if (pit != nodes_.end()) pit->second.children += 1;
        return {page, false};
    }
    void acquire(const std::vector<uint64_t>& chain) {
        for (uint64_t h : chain) nodes_.at(h).refcount += 1;
    }
    std::vector<int> release(const std::vector<uint64_t>& chain) {
        std::vector<int> freed;
        for (auto it = chain.rbegin(); it != chain.rend(); ++it) {
            auto n = nodes_.find(*it);
            if (n == nodes_.end()) continue;
            n->second.refcount -= 1;
            if (n->second.refcount <= 0 && n->second.children == 0) {
                freed.push_back(n->second.page);
                const uint64_t parent = n->second.parent;
                nodes_.erase(n);
                auto p = nodes_.find(parent);
                if (p != nodes_.end()) p->second.children -= 1;
            }
        }
        pool.free(freed);
        return freed;
    }
    int would_free(const std::vector<uint64_t>& chain) const {
        int n = 0;
        for (auto it = chain.rbegin(); it != chain.rend(); ++it) {
            auto node = nodes_.find(*it);
            if (node == nodes_.end() || node->second.refcount > 1 || node->second.children > (n ? 1 : 0)) break;
            ++n;
        }
        return n;
    }
    int prefix_len(const std::vector<uint64_t>& hashes) const {
        int n = 0;
        for (uint64_t h : hashes) {
            if (!nodes_.count(h)) break;
            ++n;
        }
        return n;
    }
    std::vector<int> physical_ids(const std::vector<uint64_t>& chain) const {
        std::vector<int> out;
        out.reserve(chain.size());
        for (uint64_t h : chain) out.push_back(nodes_.at(h).page);
        return out;
    }
    double effective_pages(const std::vector<uint64_t>& chain, int working) const {
        double s = working;
        for (uint64_t h : chain) {
            auto it = nodes_.find(h);
            if (it != nodes_.end()) s += 1.0 / (it->second.refcount > 0 ? it->second.refcount : 1);
        }
        return s;
    }
    size_t node_count() const { return nodes_.size(); }
    std::vector<int> node_pages() const {
        std::vector<int> out;
        for (auto& kv : nodes_) out.push_back(kv.second.page);
        return out;
    }

private:
    std::unordered_map<uint64_t, Node> nodes_;
};

}  // namespace pie_host
