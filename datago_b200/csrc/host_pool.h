// A small persistent pool of host threads for the per-batch planning work (header parsing, staging copies, filter
// tables).  One pool per process, created on first use and never torn down: batches are planned many times per second
// by several contexts, and spawning threads for each of them oversubscribes a host that runs one process per GPU.
//
// Size: DATAGO_B200_HOST_THREADS if set, else the cores of the host divided by the local ranks (LOCAL_WORLD_SIZE, as
// torchrun sets it) and by two (a rank normally drives two contexts), at most 8, at least 1; the calling thread
// counts as one of them.  One job runs at a time: a caller that finds the pool busy does its work on its own thread.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace dg {

class HostPool {
public:
    static HostPool& get() {
        static HostPool* pool = new HostPool();  // deliberately leaked: workers may outlive static destructors
        return *pool;
    }
    int threads() const { return (int)workers_.size() + 1; }

    // Calls fn(i) for every i in [0, n); returns when all calls have returned.  grain: fewest items worth a hand-over.
    void run(size_t n, const std::function<void(size_t)>& fn, size_t grain = 64) {
        if (n == 0) return;
        if (workers_.empty() || n < 2 * grain || !job_mu_.try_lock()) {
            for (size_t i = 0; i < n; ++i) fn(i);
            return;
        }
        const size_t parts = std::min<size_t>(threads() * 4, (n + grain - 1) / grain);
        {
            std::lock_guard<std::mutex> lock(mu_);
            fn_ = &fn;
            total_ = n;
            chunk_ = (n + parts - 1) / parts;
            next_.store(0);
            busy_ = (int)workers_.size();
            ++generation_;
        }
        cv_work_.notify_all();
        drain();
        {
            std::unique_lock<std::mutex> lock(mu_);
            cv_done_.wait(lock, [&] { return busy_ == 0; });
            fn_ = nullptr;
        }
        job_mu_.unlock();
    }

private:
    HostPool() {
        int want = 0;
        if (const char* e = getenv("DATAGO_B200_HOST_THREADS")) want = atoi(e);
        if (want <= 0) {
            int ranks = 1;
            if (const char* e = getenv("LOCAL_WORLD_SIZE")) ranks = std::max(1, atoi(e));
            const int hw = (int)std::thread::hardware_concurrency();
            want = std::max(1, std::min(8, (hw > 0 ? hw : 2) / ranks / 2));
        }
        for (int i = 1; i < std::min(want, 64); ++i) workers_.emplace_back([this] { loop(); });
        for (auto& t : workers_) t.detach();
    }
    void drain() {
        for (;;) {
            const size_t a = next_.fetch_add(chunk_);
            if (a >= total_) return;
            const size_t b = std::min(total_, a + chunk_);
            for (size_t i = a; i < b; ++i) (*fn_)(i);
        }
    }
    void loop() {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lock(mu_);
                cv_work_.wait(lock, [&] { return generation_ != seen; });
                seen = generation_;
            }
            drain();
            {
                std::lock_guard<std::mutex> lock(mu_);
                if (--busy_ == 0) cv_done_.notify_all();
            }
        }
    }

    std::vector<std::thread> workers_;
    std::mutex mu_, job_mu_;
    std::condition_variable cv_work_, cv_done_;
    const std::function<void(size_t)>* fn_ = nullptr;
    std::atomic<size_t> next_{0};
    size_t total_ = 0, chunk_ = 1;
    int busy_ = 0;
    uint64_t generation_ = 0;
};

}  // namespace dg
