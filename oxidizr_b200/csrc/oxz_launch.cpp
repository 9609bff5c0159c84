// One thread per rank with a first-failure abort: the counterpart of run_ranks (src/dp/launch.rs:183-272).
// The first rank whose body returns an error (or throws) aborts every communicator of the group once, so peers
// blocked in a collective return; every thread is joined; the error reported is the one of the rank that failed
// first, with its rank as context. Later errors follow from the abort and are dropped.
#include <atomic>
#include <cstring>
#include <exception>
#include <thread>

#include "oxz_internal.h"

using namespace oxz;

namespace {

constexpr uint64_t NO_TICKET = ~0ull;

struct FailureLog {
    std::atomic<bool> aborted{false};
    std::atomic<uint64_t> next{0};
    std::vector<std::atomic<uint64_t>> tickets;
    oxz_comm* const* comms;
    int32_t world;
    explicit FailureLog(int32_t n, oxz_comm* const* c) : tickets(n), comms(c), world(n) {
        for (auto& t : tickets) t.store(NO_TICKET);
    }
    // Record `rank`'s first failure, then abort the group once (src/dp/launch.rs:142-150).
    void fail(int32_t rank) {
        const uint64_t order = next.fetch_add(1);
        uint64_t expected = NO_TICKET;
        tickets[rank].compare_exchange_strong(expected, order);
        if (!aborted.exchange(true) && comms)
            for (int32_t r = 0; r < world; r++)
                if (comms[r]) oxz_comm_abort(comms[r]);
    }
};

struct Outcome {
    int32_t status = OXZ_OK;
    std::string message;
};

}  // namespace

extern "C" {

int32_t oxz_set_last_error(const char* message) {
    return oxz::guarded("oxz_set_last_error", [&]() -> int32_t {
        fail(OXZ_ERR_INVALID, "%s", message ? message : "");
        return OXZ_OK;
    });
}

int32_t oxz_run_ranks(int32_t world, oxz_comm* const* comms, oxz_rank_body body, void* user, int32_t* failed_rank) {
    return oxz::guarded("oxz_run_ranks", [&]() -> int32_t {
        if (failed_rank) *failed_rank = -1;
        if (!body) return fail(OXZ_ERR_INVALID, "oxz_run_ranks: null body");
        if (world < 1) return fail(OXZ_ERR_INVALID, "world size is 0: a run needs at least one rank. Pass a world size of 1 or more.");
        if (world == 1) {
            // a group of 1 runs the body on the calling thread and returns its error unchanged
            const int32_t st = body(0, 1, user);
            if (st != OXZ_OK && failed_rank) *failed_rank = 0;
            return st;
        }
        FailureLog log(world, comms);
        std::vector<Outcome> outcomes(world);
        std::vector<std::thread> threads;
        threads.reserve(world);
        for (int32_t rank = 0; rank < world; rank++) {
            try {
                threads.emplace_back([&, rank] {
                    Outcome& o = outcomes[rank];
                    try {
                        clear_error();
                        o.status = body(rank, world, user);
                        if (o.status != OXZ_OK) o.message = oxz_last_error();
                    } catch (const std::exception& e) {
                        o.status = OXZ_ERR_INVALID;
                        o.message = std::string("panic: ") + e.what();
                    } catch (...) {
                        o.status = OXZ_ERR_INVALID;
                        o.message = "panic: unknown exception";
                    }
                    if (o.status != OXZ_OK) log.fail(rank);
                });
            } catch (const std::exception& e) {
                // the started ranks would wait for this one forever
                outcomes[rank].status = OXZ_ERR_STATE;
                outcomes[rank].message = std::string("the thread of rank ") + std::to_string(rank) + " did not start: " + e.what();
                log.fail(rank);
            }
        }
        for (auto& t : threads) t.join();
        int32_t first = -1;
        for (int32_t rank = 0; rank < world; rank++) {
            if (outcomes[rank].status == OXZ_OK) continue;
            if (first < 0 || log.tickets[rank].load() < log.tickets[first].load()) first = rank;
        }
        if (first < 0) return OXZ_OK;
        if (failed_rank) *failed_rank = first;
        return fail(outcomes[first].status, "rank %d of %d failed first: %s", first, world, outcomes[first].message.c_str());
    });
}

}  // extern "C"
