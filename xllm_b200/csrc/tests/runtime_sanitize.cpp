// Stress harness for the C++ runtime, built with -fsanitize=address,undefined and with
// -fsanitize=thread by the CPU test tier (tests/test_sanitizers_cpu.py).
//
// It drives the scheduler, the block manager with its prefix cache and the virtual-memory page pool
// (host emulation) without Python: many requests with shared prefixes through chunked prefill, decode,
// preemption under a tight block budget, aborts, pause / resume; and a second thread that submits and
// aborts requests while the first one steps (the server's intake thread against the engine thread
// hand requests over under one lock, exactly as here).  Invariants are checked at the end; memory
// errors, undefined behaviour and data races are the sanitizers' part.
#include <atomic>
#include <cstdio>
#include <mutex>
#include <random>
#include <thread>

#include "scheduler.h"
#include "vmm.h"

using namespace xllm;

static int fail(const char* what) {
  std::fprintf(stderr, "FAILED: %s\n", what);
  return 1;
}

int main() {
  SchedulerConfig cfg;
  cfg.max_tokens_per_batch = 96;
  cfg.max_seqs_per_batch = 12;
  cfg.block_size = 16;
  cfg.num_blocks = 40;   // tight: forces preemption
  cfg.enable_prefix_cache = true;
  Scheduler sched(cfg);
  std::mutex mu;
  std::atomic<bool> stop{false};
  std::atomic<int> submitted{0};

  auto submit = [&](int i, std::mt19937& rng) {
    std::vector<int32_t> prompt;
    const int shared = (i % 3 == 0) ? 32 : 0;             // a third of the requests share a prefix
    for (int t = 0; t < shared; ++t) prompt.push_back(7 + t);
    const int n = 5 + (int)(rng() % 60);
    for (int t = 0; t < n; ++t) prompt.push_back((int32_t)(rng() % 1000));
    SamplingParams sp;
    StoppingParams st;
    st.max_tokens = 4 + (int)(rng() % 12);
    st.ignore_eos = true;
    std::lock_guard<std::mutex> g(mu);
    if (sched.add_request("r" + std::to_string(i), prompt, sp, st, 1, 0, 0.0, i % 5 == 0, false)) submitted++;
  };

  std::thread intake([&] {
    std::mt19937 rng(1);
    for (int i = 0; i < 120 && !stop; ++i) {
      submit(i, rng);
      if (i % 11 == 10) {
        std::lock_guard<std::mutex> g(mu);
        sched.abort_request("r" + std::to_string(i - 3));
      }
      std::this_thread::yield();
    }
  });

  std::mt19937 rng(2);
  long steps = 0, tokens = 0, finished = 0;
  for (int idle = 0; idle < 2000;) {
    std::vector<OutputEvent> evs;
    {
      std::lock_guard<std::mutex> g(mu);
      if (steps == 50) sched.pause(PauseMode::KEEP);
      if (steps == 55) sched.resume();
      auto batches = sched.schedule();
      for (auto& b : batches) {
        std::vector<int64_t> next(b.sample_rows.size());
        for (auto& t : next) t = (int64_t)(rng() % 1000);
        auto e = sched.process_output(b.batch_id, next.data(), (int64_t)next.size(), nullptr);
        evs.insert(evs.end(), e.begin(), e.end());
        tokens += b.n_tokens;
      }
      if (batches.empty()) {
        auto e = sched.take_pending_events();
        evs.insert(evs.end(), e.begin(), e.end());
      }
      idle = (batches.empty() && !sched.has_unfinished() && submitted >= 100) ? idle + 1 : (batches.empty() ? idle + 1 : 0);
    }
    for (auto& e : evs) finished += e.request_finished ? 1 : 0;
    ++steps;
    if (submitted >= 110 && finished >= submitted - 0 && idle > 5) break;
  }
  stop = true;
  intake.join();
  {
    std::lock_guard<std::mutex> g(mu);
    for (int k = 0; k < 200 && sched.has_unfinished(); ++k) {
      for (auto& b : sched.schedule()) {
        std::vector<int64_t> next(b.sample_rows.size(), 1);
        sched.process_output(b.batch_id, next.data(), (int64_t)next.size(), nullptr);
      }
    }
    if (sched.has_unfinished()) return fail("requests left unfinished");
    auto st = sched.block_manager(0).stats();
    if (st.num_free + st.num_evictable != st.num_blocks - 1) return fail("blocks leaked");
  }

  // virtual-memory page pool on its host emulation
  {
    PhyPagePool pool(fake_driver(), 0, 64 * 1024, 6);
    XTensor a(&pool, 6 * pool.page_bytes()), b(&pool, 6 * pool.page_bytes());
    a.ensure(4 * pool.page_bytes());
    reinterpret_cast<volatile char*>(a.ptr())[3 * pool.page_bytes() + 5] = 42;
    b.ensure(2 * pool.page_bytes());
    bool threw = false;
    try {
      b.ensure(3 * pool.page_bytes());
    } catch (const std::exception&) {
      threw = true;
    }
    if (!threw) return fail("pool exhaustion not reported");
    a.release_all();
    b.ensure(6 * pool.page_bytes());
    reinterpret_cast<volatile char*>(b.ptr())[5 * pool.page_bytes()] = 1;
    if (pool.pages_in_use() != 6 || pool.pages_created() != 6) return fail("page accounting");
  }
  std::printf("RUNTIME_SANITIZE_OK steps=%ld tokens=%ld finished=%ld submitted=%d\n", steps, tokens, finished, submitted.load());
  return 0;
}
