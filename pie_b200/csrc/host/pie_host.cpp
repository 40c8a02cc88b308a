// Python bindings of the native host runtime pieces: BRLE, page pool / content-addressed page
// store, BPE merge engine. Built in-tree by pie_b200._build into pie_b200/_C/pie_host*.so.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "bpe.hpp"
#include "brle.hpp"
#include "grammar.hpp"
#include "pagestore.hpp"
#include "poll_ring.hpp"
#include "shm_channel.hpp"

namespace py = pybind11;
using namespace pie_host;

PYBIND11_MODULE(pie_host, m) {
    m.doc() = "native host runtime of pie_b200";

    // ------------------------------------------------------------------ BRLE
    m.def("brle_encode", [](py::array_t<bool, py::array::c_style | py::array::forcecast> bits) {
        return brle_encode(reinterpret_cast<const uint8_t*>(bits.data()), (size_t)bits.size());
    });
    m.def("brle_decode", [](const Brle& runs, long size, bool tail) {
        const size_t n = size < 0 ? (size_t)brle_length(runs) : (size_t)size;
        py::array_t<bool> out(n);
        brle_decode(runs, reinterpret_cast<uint8_t*>(out.mutable_data()), n, tail);
        return out;
    }, py::arg("runs"), py::arg("size") = -1, py::arg("tail") = false);
    m.def("brle_and", &brle_and);
    m.def("brle_length", &brle_length);
    m.def("brle_count_true", &brle_count_true);
    m.def("brle_to_bitmask", [](const std::vector<Brle>& rows, size_t nbits, bool tail) {
        const size_t nw = (nbits + 31) / 32;
        py::array_t<uint32_t> out({rows.size(), nw});
        for (size_t r = 0; r < rows.size(); ++r) brle_to_bitmask(rows[r], out.mutable_data(r, 0), nbits, tail);
        return out;
    }, py::arg("rows"), py::arg("nbits"), py::arg("tail") = false);
    m.def("brle_droppable_pages", [](const std::vector<Brle>& rows, int page_size, int num_pages) {
        auto v = brle_droppable_pages(rows, page_size, num_pages);
        py::array_t<bool> out(v.size());
        std::copy(v.begin(), v.end(), reinterpret_cast<uint8_t*>(out.mutable_data()));
        return out;
    });

    // ------------------------------------------------------------------ runtime <-> driver channel
    py::class_<ShmChannel>(m, "ShmChannel")
        .def(py::init<const std::string&, bool, uint32_t, uint32_t, uint32_t, uint32_t, uint64_t, uint32_t>(),
             py::arg("name"), py::arg("create"), py::arg("num_slots") = 64, py::arg("req_capacity") = 1 << 20,
             py::arg("resp_capacity") = 1 << 20, py::arg("schema_version") = 0, py::arg("schema_hash") = 0,
             py::arg("spin_iters") = 2000)
        .def_property_readonly("num_slots", &ShmChannel::num_slots)
        .def_property_readonly("req_capacity", &ShmChannel::req_capacity)
        .def_property_readonly("resp_capacity", &ShmChannel::resp_capacity)
        .def_property_readonly("closed", &ShmChannel::closed)
        .def("close", &ShmChannel::close_channel)
        .def("submit", [](ShmChannel& c, py::buffer b) {
            py::buffer_info info = b.request();
            return c.submit(info.ptr, (size_t)info.size * (size_t)info.itemsize);
        })
        .def("wait_response", [](ShmChannel& c, int slot, double timeout_s) -> py::object {
            int rc;
            {
                py::gil_scoped_release nogil;
                rc = c.wait_response(slot, (uint64_t)(timeout_s * 1e9));
            }
            if (rc == 1) {
                uint32_t len;
                const uint8_t* p = c.response(slot, &len);
                py::bytes out(reinterpret_cast<const char*>(p), len);
                uint64_t q, sv;
                c.timings(slot, &q, &sv);
                c.release(slot);
                return py::make_tuple(out, (double)q * 1e-3, (double)sv * 1e-3);
            }
            if (rc == -2) throw std::runtime_error("driver channel closed");
            return py::none();
        }, py::arg("slot"), py::arg("timeout_s"))
        .def("abort", &ShmChannel::abort_slot)
        .def("slot_state", &ShmChannel::slot_state)
        .def("next_request", [](ShmChannel& c, double timeout_s) -> py::object {
            int slot;
            {
                py::gil_scoped_release nogil;
                slot = c.next_request((uint64_t)(timeout_s * 1e9));
            }
            if (slot == -2) throw std::runtime_error("driver channel closed");
            if (slot < 0) return py::none();
            uint32_t len;
            uint64_t id;
            const uint8_t* p = c.request(slot, &len, &id);
            return py::make_tuple(slot, id, py::bytes(reinterpret_cast<const char*>(p), len));
        }, py::arg("timeout_s"))
        .def("respond", [](ShmChannel& c, int slot, py::buffer b) {
            py::buffer_info info = b.request();
            return c.respond(slot, info.ptr, (size_t)info.size * (size_t)info.itemsize);
        });

    py::class_<PollRing>(m, "PollRing")
        .def(py::init<uint32_t, int64_t>(), py::arg("slots") = 1024, py::arg("spin_budget") = 20000)
        .def_property_readonly("slots", &PollRing::slots)
        .def_property_readonly("parks", &PollRing::parks)
        .def_property_readonly("closed", &PollRing::closed)
        .def_property_readonly("head", &PollRing::head)
        .def_property_readonly("tail", &PollRing::tail)
        .def("claim", &PollRing::claim)
        .def("publish", &PollRing::publish)
        .def("poll", [](PollRing& r, double timeout_s) {
            py::gil_scoped_release nogil;
            return r.poll((uint64_t)(timeout_s * 1e9));
        })
        .def("complete", &PollRing::complete)
        .def("wait_done", [](PollRing& r, uint64_t seq, double timeout_s) {
            py::gil_scoped_release nogil;
            return r.wait_done(seq, (uint64_t)(timeout_s * 1e9));
        })
        .def("is_done", &PollRing::is_done)
        .def("release", &PollRing::release)
        .def("close", &PollRing::close_ring);

    // ------------------------------------------------------------------ pages
    m.def("page_hash", [](uint64_t prev, const std::vector<uint32_t>& tokens, const std::vector<uint32_t>& positions,
                          const std::string& mask_key, uint64_t adapter_seed) {
        return page_hash(prev, tokens.data(), positions.data(), tokens.size(),
                         reinterpret_cast<const uint8_t*>(mask_key.data()), mask_key.size(), adapter_seed);
    }, py::arg("prev"), py::arg("tokens"), py::arg("positions"), py::arg("mask_key") = std::string(),
       py::arg("adapter_seed") = 0);

    py::class_<PagePool>(m, "PagePool")
        .def(py::init<int>())
        .def_property_readonly("num_pages", &PagePool::num_pages)
        .def_property_readonly("free_count", &PagePool::free_count)
        .def_property_readonly("used_count", &PagePool::used_count)
        .def_property_readonly("double_free_count", &PagePool::double_free_count)
        .def("alloc", [](PagePool& p, int n) -> py::object {
            std::vector<int> out;
            if (!p.alloc(n, out)) return py::none();
            return py::cast(out);
        })
        .def("free", [](PagePool& p, const std::vector<int>& pages) { p.free(pages); });

    py::class_<PageStore>(m, "PageStore")
        .def(py::init<int>())
        .def_readonly("pool", &PageStore::pool)
        .def("lookup", [](const PageStore& s, uint64_t h) -> py::object {
            const int p = s.lookup(h);
            return p < 0 ? py::object(py::none()) : py::object(py::int_(p));
        })
        .def("extend", &PageStore::extend)
        .def("acquire", &PageStore::acquire)
        .def("release", &PageStore::release)
        .def("would_free", &PageStore::would_free)
        .def("prefix_len", &PageStore::prefix_len)
        .def("physical_ids", &PageStore::physical_ids)
        .def("effective_pages", &PageStore::effective_pages)
        .def("node_pages", &PageStore::node_pages)
        .def_property_readonly("node_count", &PageStore::node_count);

    // ------------------------------------------------------------------ grammar
    py::class_<Grammar>(m, "Grammar")
        .def(py::init([](const std::vector<std::vector<std::vector<std::pair<int, py::bytes>>>>& rules, int root) {
            // symbol = (rule id, b"") for a reference, (-1, 32-byte class bitmap) for a byte class
            auto g = new Grammar();
            g->root = root;
            g->rules.resize(rules.size());
            for (size_t r = 0; r < rules.size(); ++r) {
                for (auto& alt : rules[r]) {
                    std::vector<GSymbol> syms;
                    for (auto& sym : alt) {
                        GSymbol gs;
                        if (sym.first >= 0) {
                            if (sym.first >= (int)rules.size()) throw std::out_of_range("rule reference out of range");
                            gs.is_rule = true;
                            gs.rule = sym.first;
                        } else {
                            const std::string bits = sym.second;
                            if (bits.size() != 32) throw std::invalid_argument("byte class must be 32 bytes");
                            for (int w = 0; w < 4; ++w) {
                                uint64_t v = 0;
                                for (int b = 0; b < 8; ++b) v |= (uint64_t)(unsigned char)bits[w * 8 + b] << (8 * b);
                                gs.cls[w] = v;
                            }
                        }
                        syms.push_back(gs);
                    }
                    g->rules[r].push_back(std::move(syms));
                }
            }
            return g;
        }))
        .def_property_readonly("num_rules", [](const Grammar& g) { return g.rules.size(); })
        .def("mask_cache_stats", [](const Grammar& g) {
            std::lock_guard<std::mutex> lock(g.mask_cache.mu);
            return py::make_tuple(g.mask_cache.hits, g.mask_cache.misses, g.mask_cache.lru.size());
        })
        .def("set_mask_cache_capacity", [](Grammar& g, size_t n) {
            std::lock_guard<std::mutex> lock(g.mask_cache.mu);
            g.mask_cache.capacity = n;
            while (g.mask_cache.lru.size() > n) {
                g.mask_cache.index.erase(g.mask_cache.lru.back().first);
                g.mask_cache.lru.pop_back();
            }
        });

    py::class_<TokenTrie>(m, "TokenTrie")
        .def(py::init([](const std::vector<int>& ids, const std::vector<py::bytes>& toks) {
            auto t = new TokenTrie();
            for (size_t i = 0; i < ids.size(); ++i) t->insert(ids[i], std::string(toks[i]));
            return t;
        }))
        .def_readonly("vocab", &TokenTrie::vocab)
        .def_property_readonly("num_nodes", [](const TokenTrie& t) { return t.nodes.size(); });

    py::class_<GrammarMatcher>(m, "GrammarMatcher")
        .def(py::init<const Grammar*, const TokenTrie*>(), py::keep_alive<1, 2>(), py::keep_alive<1, 3>())
        .def("reset", &GrammarMatcher::reset)
        .def("accept_bytes", [](GrammarMatcher& mt, const py::bytes& b) { return mt.accept_bytes(std::string(b)); })
        .def("rollback", &GrammarMatcher::rollback)
        .def("can_terminate", &GrammarMatcher::can_terminate)
        .def("is_terminated", &GrammarMatcher::is_terminated)
        .def_property_readonly("num_states", &GrammarMatcher::num_states)
        .def("next_token_mask", [](const GrammarMatcher& mt) {
            std::vector<uint8_t> a;
            mt.next_token_mask(a);
            py::array_t<bool> out(a.size());
            std::copy(a.begin(), a.end(), reinterpret_cast<uint8_t*>(out.mutable_data()));
            return out;
        })
        .def("next_token_mask_brle", [](const GrammarMatcher& mt, int vocab_size, const std::vector<int>& extra) {
            std::vector<uint8_t> a;
            mt.next_token_mask(a);
            a.resize((size_t)std::max<int>(vocab_size, (int)a.size()), 0);
            for (int id : extra)
                if (id >= 0 && id < (int)a.size()) a[id] = 1;
            return brle_encode(a.data(), a.size());
        }, py::arg("vocab_size"), py::arg("extra") = std::vector<int>());

    // ------------------------------------------------------------------ BPE
    py::class_<BpeCore>(m, "BpeCore")
        .def(py::init([](const std::vector<py::bytes>& vocab, const std::vector<int>& ids,
                         const std::vector<std::pair<py::bytes, py::bytes>>& merges, int unk_id, bool byte_fallback) {
            std::vector<std::string> v;
            v.reserve(vocab.size());
            for (auto& b : vocab) v.push_back(std::string(b));
            std::vector<std::pair<std::string, std::string>> mg;
            mg.reserve(merges.size());
            for (auto& p : merges) mg.emplace_back(std::string(p.first), std::string(p.second));
            return new BpeCore(v, ids, mg, unk_id, byte_fallback);
        }), py::arg("vocab"), py::arg("ids"), py::arg("merges"), py::arg("unk_id") = 0, py::arg("byte_fallback") = false)
        .def("encode_piece", [](BpeCore& c, const py::bytes& piece) { return c.encode_piece(std::string(piece)); })
        .def("encode_pieces", [](BpeCore& c, const std::vector<py::bytes>& pieces) {
            std::vector<std::string> ps;
            ps.reserve(pieces.size());
            for (auto& p : pieces) ps.push_back(std::string(p));
            return c.encode_pieces(ps);
        })
        .def("decode", [](const BpeCore& c, const std::vector<int>& ids) { return py::bytes(c.decode(ids)); })
        .def("token_bytes", [](const BpeCore& c, int id) { return py::bytes(c.token_bytes(id)); })
        .def_property_readonly("vocab_size", &BpeCore::vocab_size);
}
