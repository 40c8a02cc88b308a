// Shared-memory request / response channel between the runtime process and a driver process.
//
// One POSIX shared-memory segment: a 64-byte header (magic "PIE4", schema version and hash of the
// wire format, slot geometry, the request wake word) followed by N slots. A slot carries one request
// and its response: {state, response wake word, request id, lengths, three wall-clock stamps, request
// bytes, response bytes}. A client claims a free slot, writes a frame, marks it ready and bumps the
// request wake word; the server takes ready slots in request-id order, writes the response into the
// same slot and bumps the slot's wake word. Both sides wait hybrid: a bounded spin, then a futex park
// on the wake word, under a hard deadline. A client that gives up (deadline, dropped lease) marks its
// slot aborted (queued or being served); the server frees an aborted slot when it gets to it instead of
// answering, so a slot is never reused while the server may still write into it.
//
// Counterpart of driver/bridge/src/ipc.rs:1-52 (layout), :451-466 (wait), :781-900 (lease / abort).
#pragma once
#include <fcntl.h>
#include <linux/futex.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

namespace pie_host {

enum : uint32_t { SLOT_FREE = 0, SLOT_CLAIMED = 1, SLOT_READY = 2, SLOT_SERVING = 3, SLOT_DONE = 4,
                 SLOT_ABORTED_QUEUED = 5, SLOT_ABORTED_SERVING = 6 };

struct ShmHeader {
    char magic[4];
    uint32_t schema_version;
    uint64_t schema_hash;
    uint32_t num_slots;
    uint32_t req_capacity;
    uint32_t resp_capacity;
    std::atomic<uint32_t> req_wake;     // futex word: bumped on every submit and on close
    std::atomic<uint64_t> next_req_id;
    std::atomic<uint32_t> closed;
    std::atomic<uint32_t> server_waiting;
    uint8_t pad[16];
};
static_assert(sizeof(ShmHeader) == 64, "header is 64 bytes");

struct ShmSlot {
    std::atomic<uint32_t> state;
    std::atomic<uint32_t> resp_wake;    // futex word: bumped when the response is ready
    uint64_t req_id;
    uint32_t req_len;
    uint32_t resp_len;
    uint64_t t_submit_ns, t_taken_ns, t_done_ns;
    uint8_t pad[16];
};
static_assert(sizeof(ShmSlot) == 64, "slot header is 64 bytes");

inline uint64_t wall_ns() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

inline long futex_wait(std::atomic<uint32_t>* w, uint32_t expect, uint64_t timeout_ns) {
    timespec ts{(time_t)(timeout_ns / 1000000000ull), (long)(timeout_ns % 1000000000ull)};
    return syscall(SYS_futex, reinterpret_cast<uint32_t*>(w), FUTEX_WAIT, expect, &ts, nullptr, 0);
}
inline void futex_wake_all(std::atomic<uint32_t>* w) {
    syscall(SYS_futex, reinterpret_cast<uint32_t*>(w), FUTEX_WAKE, INT32_MAX, nullptr, nullptr, 0);
}

class ShmChannel {
public:
    ShmChannel(const std::string& name, bool create, uint32_t num_slots, uint32_t req_capacity, uint32_t resp_capacity,
               uint32_t schema_version, uint64_t schema_hash, uint32_t spin_iters)
        : name_(name), owner_(create), spin_(spin_iters) {
        const std::string path = "/" + name;
        if (create) {
            req_capacity = (req_capacity + 63u) & ~63u;
            resp_capacity = (resp_capacity + 63u) & ~63u;
            bytes_ = sizeof(ShmHeader) + (size_t)num_slots * (sizeof(ShmSlot) + req_capacity + resp_capacity);
            int fd = shm_open(path.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
            if (fd < 0) throw std::runtime_error("shm_open(create) " + name + ": " + std::strerror(errno));
            if (ftruncate(fd, (off_t)bytes_) != 0) {
                close(fd);
                shm_unlink(path.c_str());
                throw std::runtime_error("ftruncate: " + std::string(std::strerror(errno)));
            }
            map(fd);
            std::memset(base_, 0, bytes_);
            hdr_->schema_version = schema_version;
            hdr_->schema_hash = schema_hash;
            hdr_->num_slots = num_slots;
            hdr_->req_capacity = req_capacity;
            hdr_->resp_capacity = resp_capacity;
            hdr_->next_req_id.store(1);
            std::atomic_thread_fence(std::memory_order_release);
            std::memcpy(hdr_->magic, "PIE4", 4);      // last: an opener that sees the magic sees the rest
        } else {
            int fd = shm_open(path.c_str(), O_RDWR, 0600);
            if (fd < 0) throw std::runtime_error("shm_open " + name + ": " + std::strerror(errno));
            struct stat st;
            fstat(fd, &st);
            bytes_ = (size_t)st.st_size;
            if (bytes_ < sizeof(ShmHeader)) {
                close(fd);
                throw std::runtime_error("shared segment " + name + " is not initialised");
            }
            map(fd);
            if (std::memcmp(hdr_->magic, "PIE4", 4) != 0) {
                unmap();
                throw std::runtime_error("shared segment " + name + ": bad magic");
            }
            if (hdr_->schema_version != schema_version || hdr_->schema_hash != schema_hash) {
                unmap();
                throw std::runtime_error("shared segment " + name + ": wire schema of the peer differs");
            }
        }
    }
    ~ShmChannel() {
        unmap();
        if (owner_) shm_unlink(("/" + name_).c_str());
    }
    ShmChannel(const ShmChannel&) = delete;

    uint32_t num_slots() const { return hdr_->num_slots; }
    uint32_t req_capacity() const { return hdr_->req_capacity; }
    uint32_t resp_capacity() const { return hdr_->resp_capacity; }
    bool closed() const { return hdr_->closed.load(std::memory_order_acquire) != 0; }

    void close_channel() {
        hdr_->closed.store(1, std::memory_order_release);
        hdr_->req_wake.fetch_add(1, std::memory_order_release);
        futex_wake_all(&hdr_->req_wake);
        for (uint32_t i = 0; i < hdr_->num_slots; ++i) {
            slot(i)->resp_wake.fetch_add(1, std::memory_order_release);
            futex_wake_all(&slot(i)->resp_wake);
        }
    }

    // ---- client side -------------------------------------------------------------------------
    // Returns the slot index, -1 when every slot is in use, -2 when the channel is closed.
    int submit(const void* data, size_t len) {
        if (len > hdr_->req_capacity) throw std::length_error("request frame larger than the slot");
        if (closed()) return -2;
        for (uint32_t i = 0; i < hdr_->num_slots; ++i) {
            ShmSlot* s = slot(i);
            uint32_t expect = SLOT_FREE;
            if (!s->state.compare_exchange_strong(expect, SLOT_CLAIMED, std::memory_order_acquire)) continue;
            s->req_id = hdr_->next_req_id.fetch_add(1, std::memory_order_relaxed);
            s->req_len = (uint32_t)len;
            s->resp_len = 0;
            s->t_submit_ns = wall_ns();
            std::memcpy(req_buf(i), data, len);
            s->state.store(SLOT_READY, std::memory_order_release);
            hdr_->req_wake.fetch_add(1, std::memory_order_release);
            if (hdr_->server_waiting.load(std::memory_order_acquire)) futex_wake_all(&hdr_->req_wake);
            return (int)i;
        }
        return -1;
    }

    // 1 = response ready (read it with response()), 0 = deadline passed: the slot is marked aborted,
    // -2 = channel closed.
    int wait_response(int i, uint64_t timeout_ns) {
        ShmSlot* s = slot((uint32_t)i);
        const uint64_t deadline = wall_ns() + timeout_ns;
        for (;;) {
            const uint32_t seen = s->resp_wake.load(std::memory_order_acquire);
            for (uint32_t k = 0; k < spin_; ++k) {
                if (s->state.load(std::memory_order_acquire) == SLOT_DONE) return 1;
                __builtin_ia32_pause();
            }
            if (s->state.load(std::memory_order_acquire) == SLOT_DONE) return 1;
            if (closed()) return -2;
            const uint64_t now = wall_ns();
            if (now >= deadline) {
                abort_slot(i);
                return s->state.load(std::memory_order_acquire) == SLOT_DONE ? 1 : 0;
            }
            futex_wait(&s->resp_wake, seen, std::min<uint64_t>(deadline - now, 50000000ull));
        }
    }

    const uint8_t* response(int i, uint32_t* len) {
        *len = slot((uint32_t)i)->resp_len;
        return resp_buf((uint32_t)i);
    }
    void release(int i) { slot((uint32_t)i)->state.store(SLOT_FREE, std::memory_order_release); }

    // A client that will not read the answer. A slot still waiting for the server is freed by the server.
    void abort_slot(int i) {
        ShmSlot* s = slot((uint32_t)i);
        uint32_t st = s->state.load(std::memory_order_acquire);
        while (st == SLOT_READY || st == SLOT_SERVING) {
            const uint32_t to = st == SLOT_READY ? SLOT_ABORTED_QUEUED : SLOT_ABORTED_SERVING;
            if (s->state.compare_exchange_weak(st, to, std::memory_order_acq_rel)) return;
        }
        if (st == SLOT_DONE) return;       // answered in the meantime: the caller may still read it
    }

    // ---- server side -------------------------------------------------------------------------
    // The ready slot with the lowest request id, or -1 after the timeout, or -2 when closed.
    int next_request(uint64_t timeout_ns) {
        const uint64_t deadline = wall_ns() + timeout_ns;
        for (;;) {
            const uint32_t seen = hdr_->req_wake.load(std::memory_order_acquire);
            for (uint32_t k = 0; k <= spin_; ++k) {
                int best = -1;
                uint64_t best_id = ~0ull;
                for (uint32_t i = 0; i < hdr_->num_slots; ++i) {
                    ShmSlot* s = slot(i);
                    const uint32_t st = s->state.load(std::memory_order_acquire);
                    if (st == SLOT_READY && s->req_id < best_id) {
                        best = (int)i;
                        best_id = s->req_id;
                    } else if (st == SLOT_ABORTED_QUEUED) {      // given up before anyone took it
                        s->state.store(SLOT_FREE, std::memory_order_release);
                    }
                }
                if (best >= 0) {
                    uint32_t expect = SLOT_READY;
                    if (slot((uint32_t)best)->state.compare_exchange_strong(expect, SLOT_SERVING, std::memory_order_acq_rel)) {
                        slot((uint32_t)best)->t_taken_ns = wall_ns();
                        return best;
                    }
                    continue;                                    // aborted under us: the next scan frees it
                }
                if (hdr_->req_wake.load(std::memory_order_acquire) != seen) break;
                __builtin_ia32_pause();
            }
            if (closed()) return -2;
            const uint64_t now = wall_ns();
            if (now >= deadline) return -1;
            if (hdr_->req_wake.load(std::memory_order_acquire) != seen) continue;
            hdr_->server_waiting.store(1, std::memory_order_release);
            futex_wait(&hdr_->req_wake, seen, std::min<uint64_t>(deadline - now, 50000000ull));
            hdr_->server_waiting.store(0, std::memory_order_release);
        }
    }

    const uint8_t* request(int i, uint32_t* len, uint64_t* req_id) {
        *len = slot((uint32_t)i)->req_len;
        *req_id = slot((uint32_t)i)->req_id;
        return req_buf((uint32_t)i);
    }

    // false when the client had given up on the slot (it is freed and nothing is delivered)
    bool respond(int i, const void* data, size_t len) {
        if (len > hdr_->resp_capacity) throw std::length_error("response frame larger than the slot");
        ShmSlot* s = slot((uint32_t)i);
        if (s->state.load(std::memory_order_acquire) == SLOT_ABORTED_SERVING) {
            s->state.store(SLOT_FREE, std::memory_order_release);
            return false;
        }
        std::memcpy(resp_buf((uint32_t)i), data, len);
        s->resp_len = (uint32_t)len;
        s->t_done_ns = wall_ns();
        uint32_t expect = SLOT_SERVING;
        if (!s->state.compare_exchange_strong(expect, SLOT_DONE, std::memory_order_acq_rel)) {
            s->state.store(SLOT_FREE, std::memory_order_release);       // aborted while we were serving
            return false;
        }
        s->resp_wake.fetch_add(1, std::memory_order_release);
        futex_wake_all(&s->resp_wake);
        return true;
    }

    // (queue ns, service ns) of a slot whose response is ready
    void timings(int i, uint64_t* queued_ns, uint64_t* served_ns) {
        ShmSlot* s = slot((uint32_t)i);
        *queued_ns = s->t_taken_ns - s->t_submit_ns;
        *served_ns = s->t_done_ns - s->t_taken_ns;
    }
    uint32_t slot_state(int i) { return slot((uint32_t)i)->state.load(std::memory_order_acquire); }

private:
    void map(int fd) {
        base_ = static_cast<uint8_t*>(mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0));
        close(fd);
        if (base_ == MAP_FAILED) throw std::runtime_error("mmap: " + std::string(std::strerror(errno)));
        hdr_ = reinterpret_cast<ShmHeader*>(base_);
    }
    void unmap() {
        if (base_ && base_ != MAP_FAILED) munmap(base_, bytes_);
        base_ = nullptr;
    }
    size_t stride() const { return sizeof(ShmSlot) + hdr_->req_capacity + hdr_->resp_capacity; }
    ShmSlot* slot(uint32_t i) { return reinterpret_cast<ShmSlot*>(base_ + sizeof(ShmHeader) + (size_t)i * stride()); }
    uint8_t* req_buf(uint32_t i) { return reinterpret_cast<uint8_t*>(slot(i)) + sizeof(ShmSlot); }
    uint8_t* resp_buf(uint32_t i) { return req_buf(i) + hdr_->req_capacity; }

    std::string name_;
    bool owner_;
    uint32_t spin_;
    size_t bytes_ = 0;
    uint8_t* base_ = nullptr;
    ShmHeader* hdr_ = nullptr;
};

}  // namespace pie_host
