// Stress programs for the native host structures, meant to be built with -fsanitize=address,undefined
// and with -fsanitize=thread: the polled ring and the shared-memory channel under several producers
// (their payloads are plain memory, so the thread sanitizer checks that the rings' acquire / release
// ordering is what protects them), and the page store under a random operation mix with its invariants.
// Exit code 0 = all checks passed.
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

#include "../pagestore.hpp"
#include "../poll_ring.hpp"
#include "../shm_channel.hpp"

using namespace pie_host;

#define CHECK(cond)                                                            \
    do {                                                                       \
        if (!(cond)) {                                                         \
            std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                      \
        }                                                                      \
    } while (0)

static void poll_ring_stress() {
    constexpr uint32_t N = 64;
    constexpr int PRODUCERS = 4, PER = 4000;
    PollRing ring(N, 200);
    std::vector<uint64_t> items(N), results(N);          // plain memory, ordered by the ring only
    std::atomic<int> done{0};
    std::thread consumer([&] {
        for (int served = 0; served < PRODUCERS * PER;) {
            const int64_t seq = ring.poll(2000000000ull);
            CHECK(seq >= 0);
            results[seq % N] = items[seq % N] * 3 + 1;
            ring.complete((uint64_t)seq);
            ++served;
        }
    });
    std::vector<std::thread> producers;
    for (int p = 0; p < PRODUCERS; ++p)
        producers.emplace_back([&, p] {
            for (int i = 0; i < PER; ++i) {
                int64_t seq;
                while ((seq = ring.claim()) == -1) std::this_thread::yield();
                CHECK(seq >= 0);
                const uint64_t v = (uint64_t)p * 1000003u + (uint64_t)i;
                items[seq % N] = v;
                ring.publish((uint64_t)seq);
                CHECK(ring.wait_done((uint64_t)seq, 5000000000ull));
                CHECK(results[seq % N] == v * 3 + 1);
                ring.release((uint64_t)seq);
                done.fetch_add(1);
            }
        });
    for (auto& t : producers) t.join();
    consumer.join();
    CHECK(done.load() == PRODUCERS * PER);
    CHECK(ring.poll(1000000ull) == -1);                    // idle: times out, nothing left
    ring.close_ring();
    CHECK(ring.poll(1000000ull) == -2 && ring.claim() == -2);
}

static void shm_channel_stress() {
    const std::string name = "pie_b200_stress_" + std::to_string((long)getpid());
    ShmChannel client(name, true, 8, 256, 256, 2, 0xabcdefull, 200);
    ShmChannel server(name, false, 0, 0, 0, 2, 0xabcdefull, 200);
    constexpr int CLIENTS = 3, PER = 3000;
    std::atomic<bool> stop{false};
    std::thread srv([&] {
        while (!stop.load()) {
            const int s = server.next_request(20000000ull);
            if (s < 0) continue;
            uint32_t len;
            uint64_t id;
            const uint8_t* p = server.request(s, &len, &id);
            uint8_t out[256];
            for (uint32_t i = 0; i < len; ++i) out[i] = (uint8_t)(p[i] ^ 0x5a);
            server.respond(s, out, len);
        }
    });
    std::vector<std::thread> clients;
    for (int c = 0; c < CLIENTS; ++c)
        clients.emplace_back([&, c] {
            std::mt19937 rng(c);
            for (int i = 0; i < PER; ++i) {
                uint8_t msg[64];
                const uint32_t len = 1 + rng() % 63;
                for (uint32_t k = 0; k < len; ++k) msg[k] = (uint8_t)rng();
                int s;
                while ((s = client.submit(msg, len)) == -1) std::this_thread::yield();
                CHECK(s >= 0);
                CHECK(client.wait_response(s, 5000000000ull) == 1);
                uint32_t rl;
                const uint8_t* r = client.response(s, &rl);
                CHECK(rl == len);
                for (uint32_t k = 0; k < len; ++k) CHECK(r[k] == (uint8_t)(msg[k] ^ 0x5a));
                client.release(s);
            }
        });
    for (auto& t : clients) t.join();
    stop.store(true);
    srv.join();
    // a request nobody serves: the wait runs out, the slot is marked, the next scan frees it
    const int s = client.submit("x", 1);
    CHECK(client.wait_response(s, 2000000ull) == 0 && client.slot_state(s) == SLOT_ABORTED_QUEUED);
    CHECK(server.next_request(2000000ull) == -1 && client.slot_state(s) == SLOT_FREE);
    // a request abandoned while it is being served: the answer is dropped and the slot freed
    const int s2 = client.submit("y", 1);
    CHECK(server.next_request(2000000ull) == s2);
    client.abort_slot(s2);
    CHECK(!server.respond(s2, "z", 1) && client.slot_state(s2) == SLOT_FREE);
    client.close_channel();
    CHECK(client.submit("x", 1) == -2 && server.next_request(1000000ull) == -2);
}

static void page_store_stress() {
    PageStore store(64);
    std::mt19937 rng(7);
    struct Chain { std::vector<uint64_t> hashes; };
    std::vector<Chain> chains;
    for (int step = 0; step < 20000; ++step) {
        const int op = rng() % 3;
        if (op == 0 && store.pool.free_count() >= 4) {          // commit a chain of up to 4 pages, some shared
            Chain c;
            uint64_t prev = 0;
            const int n = 1 + rng() % 4;
            const uint32_t family = rng() % 6;                    // few families: prefixes collide and dedup
            for (int i = 0; i < n; ++i) {
                std::vector<int> pg;
                CHECK(store.pool.alloc(1, pg));
                uint32_t tok[2] = {family, (uint32_t)i}, pos[2] = {(uint32_t)(2 * i), (uint32_t)(2 * i + 1)};
                const uint64_t h = page_hash(prev, tok, pos, 2, nullptr, 0, 0);
                auto [page, dedup] = store.extend(prev, h, pg[0]);
                if (dedup) store.pool.free(pg);
                CHECK(store.lookup(h) == page);
                c.hashes.push_back(h);
                prev = h;
            }
            chains.push_back(c);
        } else if (op == 1 && !chains.empty()) {                  // release one
            const size_t k = rng() % chains.size();
            const int expect = store.would_free(chains[k].hashes);
            const auto freed = store.release(chains[k].hashes);      // returns the pages it gave back to the pool
            CHECK((int)freed.size() == expect);
            chains.erase(chains.begin() + (long)k);
        } else if (!chains.empty()) {                             // queries
            const auto& c = chains[rng() % chains.size()];
            CHECK(store.prefix_len(c.hashes) == (int)c.hashes.size());
            CHECK(store.physical_ids(c.hashes).size() == c.hashes.size());
            CHECK(store.effective_pages(c.hashes, 1) <= (double)c.hashes.size() + 1.0 + 1e-9);
        }
        CHECK(store.pool.used_count() == (int)store.node_count());      // every used page is exactly one node
    }
    for (auto& c : chains) store.release(c.hashes);
    CHECK(store.pool.used_count() == 0 && store.node_count() == 0 && store.pool.double_free_count() == 0);
    std::vector<int> pg;
    CHECK(store.pool.alloc(1, pg));
    store.pool.free(pg);
    store.pool.free(pg);                                              // the detector counts it, the pool stays sound
    CHECK(store.pool.double_free_count() == 1 && store.pool.used_count() == 0);
}

int main() {
    poll_ring_stress();
    shm_channel_stress();
    page_store_stress();
    std::puts("host stress: ok");
    return 0;
}
