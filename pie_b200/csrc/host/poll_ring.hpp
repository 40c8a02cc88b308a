// In-process polled request ring: fixed slots with a generation-tagged state machine
// (FREE -> FILLED -> TAKEN -> DONE -> FREE), a single consumer that polls the head slot with a spin
// budget before parking on a futex, and producers that wait for their own slot the same way. The
// payloads stay in the caller's language runtime (indexed by slot); only the states live here, so
// both sides can wait without holding the interpreter lock.
//
// Counterpart of runtime/src/driver/inproc_polling.rs:1-120 (1024 slots, generation tags, spin budget).
#pragma once
#include <atomic>
#include <cstdint>
#include <memory>

#include "shm_channel.hpp"

namespace pie_host {

class PollRing {
public:
    enum : uint32_t { FREE = 0, FILLED = 1, TAKEN = 2, DONE = 3 };

    PollRing(uint32_t slots, int64_t spin_budget)
        : n_(slots), spin_(spin_budget), state_(new std::atomic<uint64_t>[slots]), done_wake_(new std::atomic<uint32_t>[slots]) {
        for (uint32_t i = 0; i < slots; ++i) {
            state_[i].store(0);
            done_wake_[i].store(0);
        }
    }

    uint32_t slots() const { return n_; }
    uint64_t parks() const { return parks_.load(); }

    // Producer: the sequence number of a claimed slot, or -1 when the ring is full (the slot one lap
    // behind has not been released yet), or -2 when closed.
    int64_t claim() {
        if (closed_.load(std::memory_order_acquire)) return -2;
        for (;;) {
            uint64_t seq = tail_.load(std::memory_order_acquire);
            const uint64_t want = pack(gen(seq), FREE);
            if (state_[seq % n_].load(std::memory_order_acquire) != want) return -1;
            if (tail_.compare_exchange_weak(seq, seq + 1, std::memory_order_acq_rel)) return (int64_t)seq;
        }
    }
    void publish(uint64_t seq) {
        state_[seq % n_].store(pack(gen(seq), FILLED), std::memory_order_release);
        wake_.fetch_add(1, std::memory_order_release);
        if (parked_.load(std::memory_order_acquire)) futex_wake_all(&wake_);
    }

    // Consumer: the sequence number at the head once it is filled; -1 after timeout_ns; -2 when closed.
    int64_t poll(uint64_t timeout_ns) {
        const uint64_t deadline = wall_ns() + timeout_ns;
        const uint64_t seq = head_;
        const uint64_t want = pack(gen(seq), FILLED);
        std::atomic<uint64_t>& st = state_[seq % n_];
        for (;;) {
            const uint32_t seen = wake_.load(std::memory_order_acquire);
            for (int64_t k = 0; spin_ < 0 || k <= spin_; ++k) {
                uint64_t cur = want;
                if (st.compare_exchange_strong(cur, pack(gen(seq), TAKEN), std::memory_order_acq_rel)) {
                    ++head_;
                    return (int64_t)seq;
                }
                if (closed_.load(std::memory_order_acquire)) return -2;
                if ((k & 1023) == 1023 && wall_ns() >= deadline) return -1;
                __builtin_ia32_pause();
            }
            const uint64_t now = wall_ns();
            if (now >= deadline) return -1;
            parked_.store(1, std::memory_order_release);
            if (st.load(std::memory_order_acquire) != want && !closed_.load(std::memory_order_acquire)) {
                parks_.fetch_add(1);
                futex_wait(&wake_, seen, std::min<uint64_t>(deadline - now, 50000000ull));
            }
            parked_.store(0, std::memory_order_release);
        }
    }
    void complete(uint64_t seq) {
        state_[seq % n_].store(pack(gen(seq), DONE), std::memory_order_release);
        done_wake_[seq % n_].fetch_add(1, std::memory_order_release);
        futex_wake_all(&done_wake_[seq % n_]);
    }

    // Producer: true once the slot is done; false after the timeout (the slot stays owned by the
    // request: the consumer completes it and `release` frees it).
    bool wait_done(uint64_t seq, uint64_t timeout_ns) {
        const uint64_t deadline = wall_ns() + timeout_ns;
        const uint64_t want = pack(gen(seq), DONE);
        std::atomic<uint64_t>& st = state_[seq % n_];
        for (;;) {
            const uint32_t seen = done_wake_[seq % n_].load(std::memory_order_acquire);
            for (int k = 0; k < 4000; ++k) {
                if (st.load(std::memory_order_acquire) == want) return true;
                __builtin_ia32_pause();
            }
            if (closed_.load(std::memory_order_acquire)) return st.load(std::memory_order_acquire) == want;
            const uint64_t now = wall_ns();
            if (now >= deadline) return false;
            futex_wait(&done_wake_[seq % n_], seen, std::min<uint64_t>(deadline - now, 50000000ull));
        }
    }
    bool is_done(uint64_t seq) { return state_[seq % n_].load(std::memory_order_acquire) == pack(gen(seq), DONE); }
    // Frees the slot for the next lap.
    void release(uint64_t seq) { state_[seq % n_].store(pack(gen(seq) + 1, FREE), std::memory_order_release); }

    void close_ring() {
        closed_.store(1, std::memory_order_release);
        wake_.fetch_add(1, std::memory_order_release);
        futex_wake_all(&wake_);
        for (uint32_t i = 0; i < n_; ++i) {
            done_wake_[i].fetch_add(1, std::memory_order_release);
            futex_wake_all(&done_wake_[i]);
        }
    }
    bool closed() const { return closed_.load(std::memory_order_acquire) != 0; }
    uint64_t head() const { return head_; }
    uint64_t tail() const { return tail_.load(std::memory_order_acquire); }

private:
    uint64_t gen(uint64_t seq) const { return seq / n_; }
    static uint64_t pack(uint64_t g, uint32_t s) { return (g << 2) | s; }

    uint32_t n_;
    int64_t spin_;
    std::unique_ptr<std::atomic<uint64_t>[]> state_;      // generation << 2 | state
    std::unique_ptr<std::atomic<uint32_t>[]> done_wake_;
    std::atomic<uint64_t> tail_{0};
    uint64_t head_ = 0;                                    // consumer only
    std::atomic<uint32_t> wake_{0}, parked_{0}, closed_{0};
    std::atomic<uint64_t> parks_{0};
};

}  // namespace pie_host
