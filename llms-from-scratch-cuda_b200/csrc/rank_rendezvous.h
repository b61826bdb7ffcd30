// Host-side rendezvous of the ranks of one multi-GPU job (one process per GPU, forked from one parent).
//
// Why: a collective (NCCL) that one rank never joins leaves the other ranks waiting inside it on their
// GPUs, and a process killed there can leave more than its own GPU in a bad state.  So the ranks meet on
// the host first: every rank says "I am at collective point n" on a page of shared memory and waits, with a
// time limit, until all ranks have said so.  Only then do they enqueue the collective.  A rank that failed
// (or the parent, which sees it exit) raises the stop flag; the others notice it while they wait on the
// host, with nothing in flight on their GPUs, and leave between steps.
//
// Plain C++ (no CUDA): usable and testable on any host.  The page is created with mmap before fork().
#pragma once
#include <sys/mman.h>
#include <time.h>

#include <atomic>
#include <cstdint>
#include <new>

namespace b200 {

constexpr int kMaxRanks = 16;

struct alignas(64) RankSlot {
    std::atomic<uint64_t> arrived;   // number of collective points this rank has reached
    std::atomic<uint64_t> heartbeat; // bumped whenever the rank passes a point (diagnostics)
    char pad[64 - 2 * sizeof(std::atomic<uint64_t>)];
};

struct RendezvousPage {
    std::atomic<int> stop;           // non-zero: a rank failed; nobody starts another collective
    std::atomic<int> failed_rank;    // which one (-1: none)
    int ranks;
    char pad[64 - 3 * sizeof(int)];
    RankSlot slot[kMaxRanks];
};

enum RendezvousResult { RV_OK = 0, RV_STOPPED = 1, RV_TIMEOUT = 2 };

// Shared, zeroed page; nullptr on failure.  Call before fork().
inline RendezvousPage* rendezvous_create(int ranks) {
    if (ranks < 1 || ranks > kMaxRanks) return nullptr;
    void* p = mmap(nullptr, sizeof(RendezvousPage), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
    if (p == MAP_FAILED) return nullptr;
    RendezvousPage* page = new (p) RendezvousPage();
    page->stop.store(0);
    page->failed_rank.store(-1);
    page->ranks = ranks;
    for (int r = 0; r < kMaxRanks; ++r) {
        page->slot[r].arrived.store(0);
        page->slot[r].heartbeat.store(0);
    }
    return page;
}

inline void rendezvous_destroy(RendezvousPage* page) {
    if (page) munmap(page, sizeof(RendezvousPage));
}

inline double rendezvous_now() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

// Rank `rank` has reached its next collective point.  Returns RV_OK once every rank has reached the same
// point, RV_STOPPED if the stop flag is (or becomes) set, RV_TIMEOUT after `timeout_s` seconds -- in which case
// this rank raises the stop flag itself, naming the slowest rank, so that the others leave as well.
inline RendezvousResult rendezvous_arrive(RendezvousPage* page, int rank, double timeout_s) {
    if (page->stop.load(std::memory_order_acquire)) return RV_STOPPED;
    const uint64_t point = page->slot[rank].arrived.fetch_add(1, std::memory_order_acq_rel) + 1;
    page->slot[rank].heartbeat.fetch_add(1, std::memory_order_relaxed);
    const double t0 = rendezvous_now();
    unsigned spins = 0;
    while (true) {
        int behind = -1;
        for (int r = 0; r < page->ranks; ++r)
            if (page->slot[r].arrived.load(std::memory_order_acquire) < point) { behind = r; break; }
        if (behind < 0) return RV_OK;  // all here: everyone takes this collective, whatever happened since
        if (page->stop.load(std::memory_order_acquire)) return RV_STOPPED;
        if ((++spins & 1023u) == 0) {
            if (rendezvous_now() - t0 > timeout_s) {
                int expected = -1;
                page->failed_rank.compare_exchange_strong(expected, behind);
                page->stop.store(1, std::memory_order_release);
                return RV_TIMEOUT;
            }
            timespec nap = {0, 20000};  // 20 us: the wait is long only when something is wrong
            nanosleep(&nap, nullptr);
        }
    }
}

// Raise the stop flag (a rank that is about to exit with an error, or the parent that saw one exit).
inline void rendezvous_fail(RendezvousPage* page, int rank) {
    int expected = -1;
    page->failed_rank.compare_exchange_strong(expected, rank);
    page->stop.store(1, std::memory_order_release);
}

}  // namespace b200
