/*
 * The ring protocol on host threads: a loopback transport for tests.
 *
 * One thread per rank and plain memcpy stand in for one process per GPU and
 * the copy engines. Everything else is the protocol of
 * iris_b200_ring_attention(): at the start of call n every rank pushes its
 * rows into slot s of every consumer's pool (set n & 1) and then advances
 * the consumer's arrival word s to n; the consumer walks the steps in ring
 * order (iris_b200_ring_source), waits for each arrival word with a time
 * limit, and never sends an acknowledgement. Instead of computing attention
 * the consumer checks what it received (a header with the call number, the
 * row count and a checksum travels in front of the rows) and folds it into a
 * digest, so a run has a known answer.
 *
 * What it is for: the failure paths that must not be provoked on a GPU. The
 * caller injects faults on the host (a push that is dropped, delayed or
 * corrupted, a rank that leaves between two calls, ranks that disagree about
 * a row count) and every rank must come back with a status: ETIMEOUT for a
 * chunk that never arrives, EPROTO for one that arrives wrong. No rank may
 * block: a wait that runs out ends that rank's run. It also checks the claim
 * that two pool sets make acknowledgements unnecessary, under real thread
 * interleavings: a chunk overwritten too early fails its checksum.
 *
 * No device is touched. The reference has nothing comparable (it is single
 * device, iris_cuda.cu:122).
 */
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "iris_b200.h"

namespace {

struct Header {
    uint32_t call;
    uint32_t rows;
    uint64_t sum;
};

/* Byte b of row `row` of rank `rank` in call `call`: cheap, and different
 * for every (rank, call), so stale or foreign rows never pass for current. */
inline uint8_t pattern(int rank, uint32_t call, int row, int b) {
    uint32_t x = (uint32_t)rank * 0x9E3779B1u ^ call * 0x85EBCA77u ^ (uint32_t)row * 0xC2B2AE3Du ^ (uint32_t)b * 0x27D4EB2Fu;
    x ^= x >> 15;
    x *= 0x2C1B3C6Du;
    x ^= x >> 12;
    return (uint8_t)x;
}

inline uint64_t checksum(const uint8_t *p, size_t n) {
    uint64_t h = 1469598103934665603ull;              /* FNV-1a */
    for (size_t i = 0; i < n; i++) h = (h ^ p[i]) * 1099511628211ull;
    return h;
}

inline uint64_t fold(uint64_t digest, uint64_t chunk_sum, int step) {
    digest ^= chunk_sum + 0x9E3779B97F4A7C15ull + (digest << 6) + (digest >> 2) + (uint64_t)step;
    return digest * 0xD6E8FEB86659FD93ull;
}

void fill_rows(std::vector<uint8_t> &buf, int rank, uint32_t call, int rows, int row_bytes) {
    buf.resize((size_t)rows * row_bytes);
    for (int r = 0; r < rows; r++)
        for (int b = 0; b < row_bytes; b++) buf[(size_t)r * row_bytes + b] = pattern(rank, call, r, b);
}

struct Loop {
    int G, row_bytes, calls;
    const int *rows_of;
    size_t slot_bytes;                                  /* header + the longest chunk */
    unsigned wait_us;
    const iris_b200_loop_fault *faults;
    int nfaults;
    std::vector<std::vector<uint8_t>> pool;             /* per rank: 2 sets x G slots */
    std::vector<std::atomic<uint32_t>> arrive;          /* per rank: G words */

    const iris_b200_loop_fault *fault(int kind, int rank, int call, int step) const {
        for (int i = 0; i < nfaults; i++) {
            const iris_b200_loop_fault &f = faults[i];
            if (f.kind == kind && f.rank == rank && f.call == call && (f.step == step || f.step < 0)) return &f;
        }
        return NULL;
    }
    uint8_t *slot(int rank, uint32_t call, int s) { return pool[rank].data() + ((size_t)(call & 1u) * G + s) * slot_bytes; }
};

/* One rank's run. Returns its status; *digest covers the calls it completed. */
int run_rank(Loop &L, int me, uint64_t *digest, int *calls_done) {
    const int G = L.G;
    std::vector<uint8_t> mine;
    *digest = 0;
    *calls_done = 0;
    for (uint32_t call = 1; call <= (uint32_t)L.calls; call++) {
        if (L.fault(IRIS_B200_LOOP_LEAVE, me, (int)call, -1)) return IRIS_B200_OK;      /* gone between two calls */
        const int rows = L.rows_of[me];
        fill_rows(mine, me, call, rows, L.row_bytes);
        const uint64_t sum = checksum(mine.data(), mine.size());
        uint64_t d = *digest;                             /* committed when the call completes */
        /* All pushes, in step order, before any consumption. */
        for (int s = 1; s < G; s++) {
            const int to = (me + s) % G;
            if (L.fault(IRIS_B200_LOOP_DROP, me, (int)call, s)) continue;
            if (const iris_b200_loop_fault *f = L.fault(IRIS_B200_LOOP_DELAY, me, (int)call, s))
                std::this_thread::sleep_for(std::chrono::microseconds(f->delay_us));
            uint8_t *dst = L.slot(to, call, s);
            Header h = {call, (uint32_t)rows, sum};
            if (L.fault(IRIS_B200_LOOP_BAD_ROWS, me, (int)call, s)) h.rows += 1;
            memcpy(dst, &h, sizeof(h));
            memcpy(dst + sizeof(h), mine.data(), mine.size());
            if (L.fault(IRIS_B200_LOOP_CORRUPT, me, (int)call, s)) dst[sizeof(h) + mine.size() / 2] ^= 0x40;
            L.arrive[(size_t)to * G + s].store(call, std::memory_order_release);
        }
        /* Consumption in ring order, grouped as the attention launch groups its key parts. */
        int first[16], count[16];
        const int nparts = iris_b200_ring_plan(G, 0, first, count);
        for (int part = 0; part < nparts; part++) {
            for (int s = first[part]; s < first[part] + count[part]; s++) {
                const int src = iris_b200_ring_source(me, s, G);
                if (s == 0) {
                    d = fold(d, sum, 0);
                    continue;
                }
                std::atomic<uint32_t> &word = L.arrive[(size_t)me * G + s];
                const auto t0 = std::chrono::steady_clock::now();
                while ((int32_t)(word.load(std::memory_order_acquire) - call) < 0) {
                    if (std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(L.wait_us)) return IRIS_B200_ETIMEOUT;
                    std::this_thread::yield();
                }
                const uint8_t *p = L.slot(me, call, s);
                Header h;
                memcpy(&h, p, sizeof(h));
                if (h.call != call || (int)h.rows != L.rows_of[src]) return IRIS_B200_EPROTO;
                const uint64_t got = checksum(p + sizeof(h), (size_t)h.rows * L.row_bytes);
                if (got != h.sum) return IRIS_B200_EPROTO;
                d = fold(d, got, s);
            }
        }
        *digest = d;
        *calls_done = (int)call;
    }
    return IRIS_B200_OK;
}

}  // namespace

extern "C" int iris_b200_ring_loopback(int nranks, const int *rows_of, int row_bytes, int calls,
                                       unsigned int wait_limit_us, const iris_b200_loop_fault *faults, int nfaults,
                                       int *status_of_rank, uint64_t *digest_of_rank, int *calls_done_of_rank) {
    if (nranks < 1 || nranks > 16 || !rows_of || row_bytes <= 0 || calls < 1 || !status_of_rank || !digest_of_rank ||
        !calls_done_of_rank || (nfaults > 0 && !faults))
        return IRIS_B200_EINVAL;
    Loop L;
    L.G = nranks;
    L.row_bytes = row_bytes;
    L.calls = calls;
    L.rows_of = rows_of;
    L.wait_us = wait_limit_us ? wait_limit_us : 1000000u;
    L.faults = faults;
    L.nfaults = nfaults;
    int max_rows = 0;
    for (int r = 0; r < nranks; r++) {
        if (rows_of[r] <= 0) return IRIS_B200_EINVAL;
        max_rows = rows_of[r] > max_rows ? rows_of[r] : max_rows;
    }
    /* One row more than the longest chunk, so that a header announcing too
     * many rows is still checked inside the slot. */
    L.slot_bytes = sizeof(Header) + (size_t)(max_rows + 1) * row_bytes;
    L.pool.assign(nranks, std::vector<uint8_t>(2 * (size_t)nranks * L.slot_bytes));
    L.arrive = std::vector<std::atomic<uint32_t>>((size_t)nranks * nranks);
    for (auto &w : L.arrive) w.store(0);
    std::vector<std::thread> threads;
    for (int r = 0; r < nranks; r++)
        threads.emplace_back([&L, r, status_of_rank, digest_of_rank, calls_done_of_rank]() {
            status_of_rank[r] = run_rank(L, r, &digest_of_rank[r], &calls_done_of_rank[r]);
        });
    for (auto &t : threads) t.join();
    return IRIS_B200_OK;
}

/* The digest rank `rank` reaches after `calls` fault-free calls, computed
 * without threads, pools or waits: the known answer of a loopback run. */
extern "C" uint64_t iris_b200_ring_loopback_digest(int nranks, const int *rows_of, int row_bytes, int calls, int rank) {
    if (nranks < 1 || nranks > 16 || !rows_of || row_bytes <= 0 || rank < 0 || rank >= nranks) return 0;
    uint64_t digest = 0;
    std::vector<uint8_t> rows;
    for (uint32_t call = 1; call <= (uint32_t)calls; call++) {
        for (int s = 0; s < nranks; s++) {
            const int src = iris_b200_ring_source(rank, s, nranks);
            fill_rows(rows, src, call, rows_of[src], row_bytes);
            digest = fold(digest, checksum(rows.data(), rows.size()), s);
        }
    }
    return digest;
}
