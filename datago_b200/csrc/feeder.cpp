// Submit / wait front end: many host threads hand single samples to one GPU.
//
// datago decodes on a pool of tokio worker threads, every task calling image::load_from_memory + image_to_payload for
// its own sample (src/worker_files.rs:83-121, src/worker_wds.rs:183-227, src/worker_http.rs:276-332 of datago).  The
// GPU wants hundreds of images per launch, so this file turns those independent calls into batches: dg_submit queues
// one sample and returns a ticket, lane threads gather what is queued (up to max_batch, or whatever has arrived when
// the oldest sample has waited max_wait_us), run it through the batch entry points, and dg_wait hands each caller its
// own result.  Two lanes, each with a context of its own, keep one batch's device->host copy overlapped with the
// planning, upload and kernels of the next.  Everything here is host code layered on the public batch API.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../../include/datago_b200.h"
#include "host.h"

namespace {

using Clock = std::chrono::steady_clock;

struct Lane;

// One finished batch: keeps the device payloads and their pinned host copy alive until the last ticket lets go.
struct Flight {
    Lane* lane = nullptr;
    dg_batch* batch = nullptr;
    int pinned_index = -1;
    uint8_t* pinned = nullptr;
    std::atomic<int> refs{0};
};

struct PinnedBuf { uint8_t* ptr = nullptr; size_t size = 0; bool busy = false; };

struct Ticket {
    uint64_t id = 0;
    int state = 0;  // 0 queued, 1 taken by a lane, 2 done
    bool orphan = false, fetched = false;
    std::vector<uint8_t> bytes;
    uint32_t raw_w = 0, raw_h = 0, raw_c = 0, flags = 0;
    std::string key;
    uint8_t* host_out = nullptr;
    uint64_t host_cap = 0;
    dg_result res{};
    Flight* flight = nullptr;
    Clock::time_point t_submit;
};

struct Lane {
    dg_ctx* ctx = nullptr;
    std::thread thread;
    std::vector<PinnedBuf> pinned;     // touched by the lane thread only
    std::mutex dead_mu;
    std::vector<Flight*> dead;          // flights nobody references any more; the lane thread destroys them
};

}  // namespace

struct dg_feeder {
    int device = 0;
    dg_feeder_config cfg{};
    std::vector<std::unique_ptr<Lane>> lanes;
    std::mutex mu;
    std::condition_variable cv_work, cv_done, cv_space;
    std::deque<Ticket*> queue;
    std::unordered_map<uint64_t, std::unique_ptr<Ticket>> tickets;
    uint64_t next_id = 1;
    bool stop = false;
    dg_feeder_stats stats{};
};

namespace {

int set_error(int code, const char* msg) { return dg::dg_set_error(code, msg); }

void unref(Flight* f) {
    if (!f) return;
    if (f->refs.fetch_sub(1) == 1) {
        std::lock_guard<std::mutex> lock(f->lane->dead_mu);
        f->lane->dead.push_back(f);
    }
}

void bury(Lane& lane) {
    std::vector<Flight*> dead;
    {
        std::lock_guard<std::mutex> lock(lane.dead_mu);
        dead.swap(lane.dead);
    }
    for (Flight* f : dead) {
        if (f->batch) dg_batch_destroy(f->batch);
        if (f->pinned_index >= 0) lane.pinned[f->pinned_index].busy = false;
        delete f;
    }
}

int pinned_acquire(Lane& lane, size_t size, int* index) {
    if (size == 0) size = 256;
    int best = -1;
    for (size_t i = 0; i < lane.pinned.size(); ++i)
        if (!lane.pinned[i].busy && lane.pinned[i].size >= size && (best < 0 || lane.pinned[i].size < lane.pinned[best].size)) best = (int)i;
    if (best < 0) {
        for (size_t i = 0; i < lane.pinned.size(); ++i)  // recycle an idle buffer that is too small
            if (!lane.pinned[i].busy) { cudaFreeHost(lane.pinned[i].ptr); lane.pinned[i] = PinnedBuf(); best = (int)i; break; }
        PinnedBuf nb;
        nb.size = size + size / 4;
        if (cudaHostAlloc((void**)&nb.ptr, nb.size, cudaHostAllocDefault) != cudaSuccess) return set_error(DG_E_CUDA, "feeder: pinned host allocation failed");
        if (best >= 0) lane.pinned[best] = nb;
        else { lane.pinned.push_back(nb); best = (int)lane.pinned.size() - 1; }
    }
    lane.pinned[best].busy = true;
    *index = best;
    return DG_OK;
}

// Finish a group of tickets with one status (batch-level failure).
void fail_all(dg_feeder* f, const std::vector<Ticket*>& group, int rc) {
    std::lock_guard<std::mutex> lock(f->mu);
    for (Ticket* t : group) {
        memset(&t->res, 0, sizeof t->res);
        t->res.status = rc;
        t->state = 2;
        ++f->stats.completed; ++f->stats.failed;
        if (t->orphan) f->tickets.erase(t->id);
    }
    f->cv_done.notify_all();
}

void lane_main(dg_feeder* f, Lane* lane) {
    cudaSetDevice(f->device);
    std::vector<Ticket*> group;
    std::vector<dg_item> items;
    for (;;) {
        bury(*lane);
        group.clear();
        {
            std::unique_lock<std::mutex> lock(f->mu);
            f->cv_work.wait(lock, [&] { return f->stop || !f->queue.empty(); });
            if (f->stop) break;
            // let the batch fill up, but never keep the oldest sample waiting longer than max_wait_us
            const auto deadline = f->queue.front()->t_submit + std::chrono::microseconds(f->cfg.max_wait_us);
            while (!f->stop && f->queue.size() < f->cfg.max_batch && Clock::now() < deadline) f->cv_work.wait_until(lock, deadline);
            if (f->stop) break;
            while (!f->queue.empty() && group.size() < f->cfg.max_batch) {
                Ticket* t = f->queue.front();
                f->queue.pop_front();
                t->state = 1;
                group.push_back(t);
            }
            f->cv_space.notify_all();
            if (!f->queue.empty()) f->cv_work.notify_one();  // more than one batch is waiting: wake the other lane
        }
        if (group.empty()) continue;
        const int n = (int)group.size();
        items.assign(n, dg_item{});
        for (int i = 0; i < n; ++i) {
            Ticket* t = group[i];
            items[i].data = t->bytes.data();
            items[i].len = t->bytes.size();
            items[i].raw_w = t->raw_w; items[i].raw_h = t->raw_h; items[i].raw_c = t->raw_c; items[i].flags = t->flags;
            items[i].forced_key = t->key.empty() ? nullptr : t->key.c_str();
        }
        dg_batch* batch = nullptr;
        int rc = dg_batch_create(lane->ctx, items.data(), n, f->cfg.batch_flags, &batch);
        if (!rc) rc = dg_batch_upload(batch);
        for (Ticket* t : group) { std::vector<uint8_t>().swap(t->bytes); }  // staged: the copies are no longer needed
        if (!rc) rc = dg_batch_run(batch);
        int pin = -1;
        if (!rc) rc = pinned_acquire(*lane, dg_batch_packed_bytes(batch), &pin);
        if (!rc) rc = dg_batch_download_packed(batch, lane->pinned[pin].ptr, lane->pinned[pin].size);
        if (!rc) rc = dg_batch_sync(batch);
        if (rc) {
            if (batch) dg_batch_destroy(batch);
            if (pin >= 0) lane->pinned[pin].busy = false;
            fail_all(f, group, rc);
            continue;
        }
        Flight* fl = new Flight();
        fl->lane = lane; fl->batch = batch; fl->pinned_index = pin; fl->pinned = lane->pinned[pin].ptr;
        fl->refs.store(n + 1);  // one per ticket + this thread's own
        {
            std::lock_guard<std::mutex> lock(f->mu);
            for (int i = 0; i < n; ++i) {
                Ticket* t = group[i];
                dg_batch_result(batch, i, &t->res);
                t->state = 2;
                ++f->stats.completed;
                if (t->res.status) ++f->stats.failed;
                if (t->orphan) { f->tickets.erase(t->id); unref(fl); }
                else t->flight = fl;
            }
            ++f->stats.batches;
            f->stats.batched_items += (uint64_t)n;
            if ((uint32_t)n > f->stats.largest_batch) f->stats.largest_batch = (uint32_t)n;
            f->cv_done.notify_all();
        }
        unref(fl);
    }
    bury(*lane);
}

}  // namespace

extern "C" int dg_feeder_create(int device, const dg_image_config* image_config, const dg_feeder_config* config, dg_feeder** out) {
    if (!out) return set_error(DG_E_INVALID, "out is NULL");
    *out = nullptr;
    if (device == DG_DEVICE_NONE) return set_error(DG_E_INVALID, "a feeder needs a CUDA device (there is no CPU path)");
    std::unique_ptr<dg_feeder> f(new dg_feeder());
    f->device = device;
    if (config) f->cfg = *config;
    if (f->cfg.lanes == 0) f->cfg.lanes = 2;
    if (f->cfg.lanes > 8) return set_error(DG_E_INVALID, "feeder: at most 8 lanes");
    if (f->cfg.max_batch == 0) f->cfg.max_batch = 512;
    if (f->cfg.max_wait_us == 0) f->cfg.max_wait_us = 2000;
    if (f->cfg.queue_limit == 0) f->cfg.queue_limit = 4 * f->cfg.max_batch;
    if (f->cfg.batch_flags & ~(uint32_t)DG_BATCH_DECODE_ONLY) return set_error(DG_E_INVALID, "feeder: batch_flags may only hold DG_BATCH_DECODE_ONLY");
    for (uint32_t i = 0; i < f->cfg.lanes; ++i) {
        std::unique_ptr<Lane> lane(new Lane());
        const int rc = dg_ctx_create(device, image_config, &lane->ctx);
        if (rc) {
            for (auto& l : f->lanes) dg_ctx_destroy(l->ctx);
            return rc;
        }
        f->lanes.push_back(std::move(lane));
    }
    for (auto& l : f->lanes) l->thread = std::thread(lane_main, f.get(), l.get());
    *out = f.release();
    return DG_OK;
}

extern "C" const dg_ctx* dg_feeder_ctx(const dg_feeder* f) { return f && !f->lanes.empty() ? f->lanes[0]->ctx : nullptr; }

extern "C" int dg_submit(dg_feeder* f, const dg_item* item, uint8_t* host_out, uint64_t host_capacity, dg_ticket* ticket) {
    if (!f || !item || !ticket) return set_error(DG_E_INVALID, "NULL argument");
    *ticket = 0;
    if (!item->data) return set_error(DG_E_INVALID, "item has no data");
    if (item->raw_w && item->len < (uint64_t)item->raw_w * item->raw_h * item->raw_c) return set_error(DG_E_INVALID, "raw item shorter than its size says");
    std::unique_ptr<Ticket> t(new Ticket());
    t->bytes.assign(item->data, item->data + item->len);  // the caller's buffer is free again when this call returns
    t->raw_w = item->raw_w; t->raw_h = item->raw_h; t->raw_c = item->raw_c; t->flags = item->flags;
    if (item->forced_key) t->key = item->forced_key;
    t->host_out = host_out; t->host_cap = host_capacity;
    std::unique_lock<std::mutex> lock(f->mu);
    f->cv_space.wait(lock, [&] { return f->stop || f->queue.size() < f->cfg.queue_limit; });
    if (f->stop) return set_error(DG_E_INVALID, "feeder is shutting down");
    t->id = f->next_id++;
    t->t_submit = Clock::now();
    *ticket = t->id;
    f->queue.push_back(t.get());
    f->tickets.emplace(t->id, std::move(t));
    ++f->stats.submitted;
    if (f->queue.size() == 1 || f->queue.size() >= f->cfg.max_batch) f->cv_work.notify_all();
    return DG_OK;
}

static int copy_out(Ticket* t, Flight* fl, uint8_t* dst, uint64_t cap) {
    if (t->res.status) return DG_OK;  // nothing to copy; the status travels in the result
    if (cap < t->res.nbytes) return set_error(DG_E_INVALID, "host buffer smaller than the payload");
    memcpy(dst, fl->pinned + t->res.packed_offset, t->res.nbytes);
    return DG_OK;
}

extern "C" int dg_wait(dg_feeder* f, dg_ticket id, uint64_t timeout_ns, dg_result* out) {
    if (!f) return set_error(DG_E_INVALID, "NULL feeder");
    Ticket* t = nullptr;
    Flight* fl = nullptr;
    bool copy = false;
    {
        std::unique_lock<std::mutex> lock(f->mu);
        auto it = f->tickets.find(id);
        if (it == f->tickets.end() || it->second->orphan) return set_error(DG_E_INVALID, "unknown ticket");
        t = it->second.get();
        const auto done = [&] { return t->state == 2 || f->stop; };
        if (timeout_ns == UINT64_MAX) f->cv_done.wait(lock, done);
        else if (!f->cv_done.wait_for(lock, std::chrono::nanoseconds(timeout_ns), done)) return set_error(DG_E_TIMEOUT, "ticket not finished yet");
        if (t->state != 2) return set_error(DG_E_INVALID, "feeder shut down before the sample ran");
        fl = t->flight;
        copy = t->host_out && !t->fetched && fl;
        if (copy) t->fetched = true;
    }
    // Only this ticket's owner touches it from here on (releasing a ticket another thread is waiting on is a caller bug).
    int rc = DG_OK;
    if (copy) {
        rc = copy_out(t, fl, t->host_out, t->host_cap);  // on the caller's thread: the copies of a batch run in parallel
        if (!rc) {  // host path: the device copy is not needed any more, let the batch go as soon as its peers agree
            std::lock_guard<std::mutex> lock(f->mu);
            t->flight = nullptr;
            t->res.device_data = nullptr;
            unref(fl);
        }
    }
    if (out) *out = t->res;
    return rc;
}

extern "C" int dg_fetch(dg_feeder* f, dg_ticket id, uint8_t* host_out, uint64_t capacity) {
    if (!f || !host_out) return set_error(DG_E_INVALID, "NULL argument");
    Ticket* t = nullptr;
    Flight* fl = nullptr;
    {
        std::lock_guard<std::mutex> lock(f->mu);
        auto it = f->tickets.find(id);
        if (it == f->tickets.end() || it->second->orphan) return set_error(DG_E_INVALID, "unknown ticket");
        t = it->second.get();
        if (t->state != 2) return set_error(DG_E_INVALID, "ticket not finished: call dg_wait first");
        fl = t->flight;
        if (t->res.status == DG_OK && !fl) return set_error(DG_E_INVALID, "payload already handed over (host buffer given at submit)");
    }
    return copy_out(t, fl, host_out, capacity);
}

extern "C" int dg_peek(dg_feeder* f, dg_ticket id, const uint8_t** host_data) {
    if (!f || !host_data) return set_error(DG_E_INVALID, "NULL argument");
    *host_data = nullptr;
    std::lock_guard<std::mutex> lock(f->mu);
    auto it = f->tickets.find(id);
    if (it == f->tickets.end() || it->second->orphan) return set_error(DG_E_INVALID, "unknown ticket");
    const Ticket* t = it->second.get();
    if (t->state != 2) return set_error(DG_E_INVALID, "ticket not finished: call dg_wait first");
    if (t->res.status) return set_error(t->res.status, "the sample failed: there is no payload");
    if (!t->flight) return set_error(DG_E_INVALID, "payload already handed over (host buffer given at submit)");
    *host_data = t->flight->pinned + t->res.packed_offset;
    return DG_OK;
}

extern "C" int dg_release(dg_feeder* f, dg_ticket id) {
    if (!f) return set_error(DG_E_INVALID, "NULL feeder");
    std::lock_guard<std::mutex> lock(f->mu);
    auto it = f->tickets.find(id);
    if (it == f->tickets.end() || it->second->orphan) return set_error(DG_E_INVALID, "unknown ticket");
    Ticket* t = it->second.get();
    if (t->state == 2) {
        unref(t->flight);
        f->tickets.erase(it);
    } else if (t->state == 0) {  // still queued: take it out, nothing ran
        for (auto q = f->queue.begin(); q != f->queue.end(); ++q)
            if (*q == t) { f->queue.erase(q); break; }
        f->tickets.erase(it);
        f->cv_space.notify_all();
    } else {
        t->orphan = true;  // a lane is working on it; the lane drops it when the batch is done
        t->host_out = nullptr;
    }
    return DG_OK;
}

extern "C" int dg_feeder_get_stats(dg_feeder* f, dg_feeder_stats* out) {
    if (!f || !out) return set_error(DG_E_INVALID, "NULL argument");
    std::lock_guard<std::mutex> lock(f->mu);
    *out = f->stats;
    out->queued = (uint32_t)f->queue.size();
    out->open_tickets = (uint32_t)f->tickets.size();
    return DG_OK;
}

extern "C" void dg_feeder_destroy(dg_feeder* f) {
    if (!f) return;
    {
        std::lock_guard<std::mutex> lock(f->mu);
        f->stop = true;
        f->cv_work.notify_all();
        f->cv_done.notify_all();
        f->cv_space.notify_all();
    }
    for (auto& l : f->lanes) if (l->thread.joinable()) l->thread.join();
    // tickets never released: drop what they hold (device payloads die with the feeder)
    for (auto& kv : f->tickets) {
        Flight* fl = kv.second->flight;
        if (fl && fl->refs.fetch_sub(1) == 1) fl->lane->dead.push_back(fl);
    }
    f->tickets.clear();
    cudaSetDevice(f->device);
    for (auto& l : f->lanes) {
        bury(*l);
        for (PinnedBuf& p : l->pinned) if (p.ptr) cudaFreeHost(p.ptr);
        dg_ctx_destroy(l->ctx);
    }
    delete f;
}
