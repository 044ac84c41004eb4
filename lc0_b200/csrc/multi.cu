// One batch over several GPUs of the box: positions are independent, so the batch is cut into contiguous, nearly
// equal slices (sizes differ by at most one), one per GPU, with the weights replicated and no exchange step.
//
// What the reference's `demux` decorator does around per-GPU backends (DemuxingComputation::ComputeBlocking,
// src/neural/backends/network_demux.cc:279-334: the batch is split into work items that the backends' worker threads
// evaluate through their own computations), without the decorator's per-slice NewComputation and plane moves: one
// persistent host thread per GPU calls b200_net_eval_host on its slice and writes the results straight into the
// caller's arrays at the slice's offset.  Host code only; it drives the C ABI of include/b200nn.h.
#include <condition_variable>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/b200nn.h"
#include "common.cuh"

struct b200_multi {
  struct Job {
    const uint64_t* masks = nullptr;
    const float* values = nullptr;
    int n = 0;
    float *policy = nullptr, *q = nullptr, *d = nullptr, *m = nullptr;
  };
  std::vector<b200_net*> nets;
  std::vector<std::thread> workers;
  std::mutex mu, eval_mu;
  std::condition_variable cv_work, cv_done;
  std::vector<Job> jobs;        // one per GPU for the evaluation in progress
  std::vector<int> state;       // 0 idle, 1 job posted, 2 done
  std::vector<int> rc;
  std::vector<std::string> err;
  bool quit = false;

  void worker(int i) {
    for (;;) {
      Job job;
      {
        std::unique_lock<std::mutex> lock(mu);
        cv_work.wait(lock, [&] { return quit || state[i] == 1; });
        if (quit) return;
        job = jobs[i];
      }
      int r = B200_OK;
      std::string e;
      if (job.n > 0) {
        r = b200_net_eval_host(nets[i], job.masks, job.values, job.n, job.policy, job.q, job.d, job.m);
        if (r != B200_OK) e = b200_last_error();  // the error text is per thread: carry it to the caller
      }
      {
        std::lock_guard<std::mutex> lock(mu);
        rc[i] = r;
        err[i] = e;
        state[i] = 2;
      }
      cv_done.notify_all();
    }
  }
};

extern "C" {

void b200_multi_slice(int n, int parts, int part, int* begin, int* count) {
  // contiguous slices whose sizes differ by at most one position: the first n % parts slices take the extra one
  if (parts < 1) parts = 1;
  if (n < 0) n = 0;
  const int base = n / parts, extra = n % parts;
  if (begin) *begin = part * base + (part < extra ? part : extra);
  if (count) *count = base + (part < extra ? 1 : 0);
}

int b200_multi_create(const b200_builder* b, const b200_net_options* opt, const int* gpus, int n_gpus,
                      b200_multi** out) {
  if (!b || !opt || !gpus || n_gpus < 1 || n_gpus > 64 || !out) {
    b200::set_error("b200_multi_create: bad argument");
    return B200_ERR_INVALID;
  }
  b200_multi* mg = new b200_multi();
  for (int i = 0; i < n_gpus; ++i) {
    b200_net_options o = *opt;
    o.gpu = gpus[i];
    b200_net* net = nullptr;
    const int r = b200_net_create(b, &o, &net);
    if (r != B200_OK) {
      for (b200_net* made : mg->nets) b200_net_destroy(made);
      delete mg;
      return r;
    }
    mg->nets.push_back(net);
  }
  mg->jobs.resize(n_gpus);
  mg->state.assign(n_gpus, 0);
  mg->rc.assign(n_gpus, B200_OK);
  mg->err.resize(n_gpus);
  for (int i = 0; i < n_gpus; ++i) mg->workers.emplace_back([mg, i] { mg->worker(i); });
  *out = mg;
  return B200_OK;
}

int b200_multi_gpu_count(const b200_multi* mg) { return mg ? (int)mg->nets.size() : 0; }

b200_net* b200_multi_net(b200_multi* mg, int i) {
  return mg && i >= 0 && i < (int)mg->nets.size() ? mg->nets[i] : nullptr;
}

int b200_multi_eval_host(b200_multi* mg, const uint64_t* masks, const float* values, int n, float* policy, float* q,
                         float* d, float* m) {
  if (!mg || n < 0 || (n > 0 && (!masks || !values))) {
    b200::set_error("b200_multi_eval_host: bad argument");
    return B200_ERR_INVALID;
  }
  std::lock_guard<std::mutex> one_at_a_time(mg->eval_mu);
  const int parts = (int)mg->nets.size();
  {
    std::lock_guard<std::mutex> lock(mg->mu);
    for (int i = 0; i < parts; ++i) {
      int begin = 0, count = 0;
      b200_multi_slice(n, parts, i, &begin, &count);
      b200_multi::Job& j = mg->jobs[i];
      j.masks = masks + (size_t)begin * 112;
      j.values = values + (size_t)begin * 112;
      j.n = count;
      j.policy = policy ? policy + (size_t)begin * 1858 : nullptr;
      j.q = q ? q + begin : nullptr;
      j.d = d ? d + begin : nullptr;
      j.m = m ? m + begin : nullptr;
      mg->state[i] = 1;
    }
  }
  mg->cv_work.notify_all();
  int result = B200_OK;
  {
    std::unique_lock<std::mutex> lock(mg->mu);
    mg->cv_done.wait(lock, [&] {
      for (int s : mg->state)
        if (s != 2) return false;
      return true;
    });
    for (int i = 0; i < parts; ++i) {
      if (mg->rc[i] != B200_OK && result == B200_OK) {
        result = mg->rc[i];
        b200::set_error("gpu slice " + std::to_string(i) + ": " + mg->err[i]);
      }
      mg->state[i] = 0;
    }
  }
  return result;
}

void b200_multi_destroy(b200_multi* mg) {
  if (!mg) return;
  {
    std::lock_guard<std::mutex> lock(mg->mu);
    mg->quit = true;
  }
  mg->cv_work.notify_all();
  for (auto& t : mg->workers) t.join();
  for (b200_net* net : mg->nets) b200_net_destroy(net);
  delete mg;
}

}  // extern "C"
