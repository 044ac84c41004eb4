// Batch aggregation across caller threads: many small evaluation requests, one GPU batch.
//
// What the reference's `multiplexing` decorator does for any backend (MuxingNetwork::Worker,
// src/neural/backends/network_mux.cc:169-205): callers enqueue their inputs and block; worker threads gather queued
// requests into one upstream computation up to a batch limit, run it, and hand every caller its slice of the results.
// Differences, sized for a GPU whose throughput only saturates near a thousand positions per batch: a worker that
// finds the queue short waits up to `wait_us` for more requests before it launches, and two workers alternate so
// that one gathers and copies while the other's batch is on the GPU.  Host code only; it drives the C ABI of
// include/b200nn.h like any other caller.
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/b200nn.h"
#include "common.cuh"

namespace {

struct Request {
  const uint64_t* masks;
  const float* values;
  int n;
  float *policy, *q, *d, *m;
  int rc = B200_OK;
  std::string error;
  bool done = false;
};

}  // namespace

struct b200_mux {
  b200_net* net = nullptr;
  int max_batch = 0;
  int wait_us = 0;
  std::mutex mu;
  std::condition_variable cv_work, cv_done, cv_idle;
  std::deque<Request*> queue;
  int queued_positions = 0;
  int inside = 0;  // callers blocked in b200_mux_eval
  bool abort = false;
  long long batches = 0, positions = 0, requests = 0;
  std::vector<std::thread> workers;

  void worker() {
    for (;;) {
      std::vector<Request*> taken;
      int total = 0;
      {
        std::unique_lock<std::mutex> lock(mu);
        cv_work.wait(lock, [&] { return abort || !queue.empty(); });
        if (abort) return;
        // A short queue may still grow: give concurrent callers `wait_us` to arrive before launching.
        if (queued_positions < max_batch && wait_us > 0) {
          const auto deadline = std::chrono::steady_clock::now() + std::chrono::microseconds(wait_us);
          cv_work.wait_until(lock, deadline, [&] { return abort || queued_positions >= max_batch; });
          if (abort) return;
        }
        while (!queue.empty()) {
          Request* r = queue.front();
          if (total != 0 && total + r->n > max_batch) break;  // as in the reference: an oversized single request still goes
          taken.push_back(r);
          total += r->n;
          queued_positions -= r->n;
          queue.pop_front();
        }
        if (taken.empty()) continue;  // another worker took everything while this one waited
        batches++;
        positions += total;
      }
      run(taken);
      {
        std::lock_guard<std::mutex> lock(mu);
        for (Request* r : taken) r->done = true;
      }
      cv_done.notify_all();
    }
  }

  // One upstream computation for all taken requests.
  void run(const std::vector<Request*>& taken) {
    b200_comp* comp = nullptr;
    int rc = b200_comp_create(net, &comp);
    for (size_t i = 0; rc == B200_OK && i < taken.size(); ++i)
      rc = b200_comp_add_inputs(comp, taken[i]->masks, taken[i]->values, taken[i]->n);
    if (rc == B200_OK) rc = b200_comp_compute(comp);
    if (rc != B200_OK) {
      const std::string msg = b200_last_error();
      for (Request* r : taken) {
        r->rc = rc;
        r->error = msg;
      }
    } else {
      int base = 0;
      for (Request* r : taken) {
        if (r->policy && r->n > 0) memcpy(r->policy, b200_comp_policy(comp, base), (size_t)r->n * 1858 * sizeof(float));
        for (int i = 0; i < r->n; ++i) {
          if (r->q) r->q[i] = b200_comp_q(comp, base + i);
          if (r->d) r->d[i] = b200_comp_d(comp, base + i);
          if (r->m) r->m[i] = b200_comp_m(comp, base + i);
        }
        base += r->n;
      }
    }
    if (comp) b200_comp_destroy(comp);
  }
};

extern "C" {

int b200_mux_create(b200_net* net, int max_batch, int wait_us, b200_mux** out) {
  b200_net_info info;
  if (!net || !out || max_batch < 1 || wait_us < 0 || b200_net_get_info(net, &info) != B200_OK) {
    b200::set_error("b200_mux_create: bad argument");
    return B200_ERR_INVALID;
  }
  if (max_batch > info.max_batch) {
    b200::set_error("b200_mux_create: max_batch exceeds the network's max_batch=" + std::to_string(info.max_batch));
    return B200_ERR_INVALID;
  }
  b200_mux* m = new b200_mux;
  m->net = net;
  m->max_batch = max_batch;
  m->wait_us = wait_us;
  for (int i = 0; i < 2; ++i) m->workers.emplace_back([m] { m->worker(); });
  *out = m;
  return B200_OK;
}

int b200_mux_eval(b200_mux* mux, const uint64_t* masks, const float* values, int n, float* policy, float* q, float* d,
                  float* m) {
  if (!mux || n < 0 || (n > 0 && (!masks || !values)) || n > mux->max_batch) {
    b200::set_error("b200_mux_eval: bad argument (at most max_batch positions per request)");
    return B200_ERR_INVALID;
  }
  if (n == 0) return B200_OK;
  Request r{masks, values, n, policy, q, d, m};
  {
    std::unique_lock<std::mutex> lock(mux->mu);
    if (mux->abort) {
      b200::set_error("b200_mux_eval: the aggregator is being destroyed");
      return B200_ERR_INVALID;
    }
    mux->queue.push_back(&r);
    mux->queued_positions += n;
    mux->requests++;
    mux->inside++;
    mux->cv_work.notify_all();
    mux->cv_done.wait(lock, [&] { return r.done; });
    // b200_mux_destroy waits for this count to reach zero before it frees the mutex this thread still holds
    if (--mux->inside == 0) mux->cv_idle.notify_all();
  }
  if (r.rc != B200_OK) b200::set_error(r.error);
  return r.rc;
}

int b200_mux_stats(b200_mux* mux, long long* requests, long long* batches, long long* positions) {
  if (!mux) return B200_ERR_INVALID;
  std::lock_guard<std::mutex> lock(mux->mu);
  if (requests) *requests = mux->requests;
  if (batches) *batches = mux->batches;
  if (positions) *positions = mux->positions;
  return B200_OK;
}

void b200_mux_destroy(b200_mux* mux) {
  if (!mux) return;
  {
    std::lock_guard<std::mutex> lock(mux->mu);
    mux->abort = true;
    // callers still queued get an error instead of waiting for ever (the reference notifies them the same way)
    for (Request* r : mux->queue) {
      r->rc = B200_ERR_INVALID;
      r->error = "the aggregator was destroyed before the request ran";
      r->done = true;
    }
    mux->queue.clear();
  }
  mux->cv_work.notify_all();
  mux->cv_done.notify_all();
  for (auto& t : mux->workers) t.join();
  {
    // callers that were woken above are still inside b200_mux_eval until they have re-acquired and released the mutex
    std::unique_lock<std::mutex> lock(mux->mu);
    mux->cv_idle.wait(lock, [&] { return mux->inside == 0; });
  }
  delete mux;
}

}  // extern "C"
