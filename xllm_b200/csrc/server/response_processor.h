// Native response pipeline: turns the engine's output events into OpenAI completion / chat
// responses (SSE chunks or one JSON body) on worker threads, without the interpreter.
//
// Parity: AsyncResponseProcessor (xllm/core/scheduler/async_response_processor.cpp:86-376): the
// scheduler thread only enqueues (request, token) pairs; a pool of threads detokenises
// incrementally, checks stop strings, formats the chunk and hands it to the connection.  Events of
// one request always go to the same worker (handle modulo pool size), which keeps their order.
//
// The engine loop calls push() once per step with every event of the step; a call that needs more
// than text (tool-call / reasoning parsers, logprobs, the Anthropic format) stays on the
// interpreter path and is never opened here.
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../frontend/json.h"
#include "../frontend/text.h"
#include "http_server.h"
#include "metrics.h"

namespace xllm {

struct RespCallSpec {
  int64_t http_id = 0;
  std::string request_id, model;
  int kind = 0;                 // 0 text completion, 1 chat completion
  bool stream = false, include_usage = false, return_token_ids = false;
  int n = 1;
  int prompt_tokens = 0;
  int64_t created = 0;
  std::string echo_text;
  std::vector<std::string> stops;
  bool skip_special = true;
  double t_arrival = 0;         // seconds, steady clock of the caller (time.monotonic())
};

struct RespEvent {
  int64_t call = 0;
  int32_t seq_index = 0;
  int32_t token = -1;
  bool finished = false, request_finished = false, aborted = false;
  std::string finish_reason;
};

struct RespDone {
  std::string request_id;
  int64_t http_id = 0;
  int64_t generated = 0;
  int prompt_tokens = 0;
  bool aborted = false;
  double ttft_ms = 0, e2e_ms = 0;
};

class ResponseProcessor {
 public:
  ResponseProcessor(HttpServer* http, std::shared_ptr<BpeTokenizer> tok, int n_threads)
      : http_(http), tok_(std::move(tok)), workers_(n_threads < 1 ? 1 : n_threads) {
    for (size_t i = 0; i < workers_.size(); ++i) {
      workers_[i] = std::make_unique<Worker>();
      workers_[i]->thread = std::thread([this, i] { run(*workers_[i]); });
    }
  }
  ~ResponseProcessor() { stop(); }

  void stop() {
    if (stopped_.exchange(true)) return;
    for (auto& w : workers_) {
      { std::lock_guard<std::mutex> lk(w->mu); w->quit = true; }
      w->cv.notify_all();
    }
    for (auto& w : workers_)
      if (w->thread.joinable()) w->thread.join();
  }

  int64_t open(const RespCallSpec& spec) {
    auto c = std::make_shared<Call>();
    c->spec = spec;
    c->texts.assign(spec.n, std::string());
    c->ids.assign(spec.n, std::vector<int32_t>());
    c->finish.assign(spec.n, std::string());
    for (int i = 0; i < spec.n; ++i)
      c->decoders.emplace_back(tok_ ? new IncrementalDecoder(tok_.get(), spec.stops, spec.skip_special) : nullptr);
    const int64_t h = next_handle_.fetch_add(1);
    Worker& w = *workers_[(size_t)h % workers_.size()];
    { std::lock_guard<std::mutex> lk(w.mu); w.calls.emplace(h, std::move(c)); }
    return h;
  }

  // All events of one engine step.  Never blocks on formatting or on a socket.
  void push(std::vector<RespEvent> events) {
    pending_.fetch_add((int64_t)events.size());
    std::vector<bool> touched(workers_.size(), false);
    for (auto& e : events) {
      const size_t wi = (size_t)e.call % workers_.size();
      Worker& w = *workers_[wi];
      { std::lock_guard<std::mutex> lk(w.mu); w.queue.push_back(std::move(e)); }
      touched[wi] = true;
    }
    for (size_t i = 0; i < workers_.size(); ++i)
      if (touched[i]) workers_[i]->cv.notify_one();
  }

  std::vector<RespDone> take_done() {
    std::lock_guard<std::mutex> lk(done_mu_);
    std::vector<RespDone> out;
    out.swap(done_);
    return out;
  }
  int64_t pending() const { return pending_.load(); }
  int64_t processed() const { return processed_.load(); }
  int num_threads() const { return (int)workers_.size(); }

  // Blocks until every pushed event has been turned into output (tests, shutdown).
  bool drain(int timeout_ms) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    while (pending_.load() > 0) {
      if (std::chrono::steady_clock::now() > deadline) return false;
      std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    return true;
  }

 private:
  struct Call {
    RespCallSpec spec;
    std::vector<std::unique_ptr<IncrementalDecoder>> decoders;
    std::vector<std::string> texts;
    std::vector<std::vector<int32_t>> ids;
    std::vector<std::string> finish;
    bool started = false;
    double t_first = 0;
  };
  struct Worker {
    std::thread thread;
    std::mutex mu;
    std::condition_variable cv;
    std::deque<RespEvent> queue;
    std::unordered_map<int64_t, std::shared_ptr<Call>> calls;
    bool quit = false;
  };

  static double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
  }

  void run(Worker& w) {
    std::deque<RespEvent> batch;
    while (true) {
      {
        std::unique_lock<std::mutex> lk(w.mu);
        w.cv.wait(lk, [&] { return w.quit || !w.queue.empty(); });
        if (w.queue.empty() && w.quit) return;
        batch.swap(w.queue);
      }
      for (auto& e : batch) {
        std::shared_ptr<Call> c;
        {
          std::lock_guard<std::mutex> lk(w.mu);
          auto it = w.calls.find(e.call);
          if (it != w.calls.end()) c = it->second;
        }
        if (c) {
          try {
            if (handle(*c, e)) {
              std::lock_guard<std::mutex> lk(w.mu);
              w.calls.erase(e.call);
            }
          } catch (const std::exception&) {
            // a formatting failure ends this call only
            http_->respond(c->spec.http_id, 500, "application/json",
                           "{\"error\":{\"message\":\"response processing failed\",\"type\":\"internal_error\",\"code\":500}}");
            std::lock_guard<std::mutex> lk(w.mu);
            w.calls.erase(e.call);
          }
        }
        processed_.fetch_add(1);
        pending_.fetch_sub(1);
      }
      batch.clear();
    }
  }

  // ---- formatting
  static void q(std::string& out, const std::string& s) { Json::escape_to(out, s); }

  std::string head(const Call& c, const char* object) const {
    std::string o = "{\"id\":";
    q(o, c.spec.request_id);
    o += ",\"object\":\"";
    o += object;
    o += "\",\"created\":" + std::to_string(c.spec.created) + ",\"model\":";
    q(o, c.spec.model);
    return o;
  }

  // one SSE chunk; `finish` empty = null
  void sse_chunk(const Call& c, int i, const std::string& text, bool role, const std::string& finish, bool empty_delta) {
    std::string o = "data: " + head(c, c.spec.kind == 0 ? "text_completion" : "chat.completion.chunk");
    o += ",\"choices\":[{\"index\":" + std::to_string(i);
    if (c.spec.kind == 0) {
      o += ",\"text\":";
      q(o, text);
    } else {
      o += ",\"delta\":{";
      if (role) {
        o += "\"role\":\"assistant\",\"content\":\"\"";
      } else if (!empty_delta) {
        o += "\"content\":";
        q(o, text);
      }
      o += "}";
    }
    o += ",\"finish_reason\":";
    if (finish.empty()) o += "null"; else q(o, finish);
    o += "}]}\n\n";
    http_->stream_send(c.spec.http_id, o);
  }

  void start_stream(Call& c) {
    c.started = true;
    http_->stream_begin(c.spec.http_id, 200, "text/event-stream");
    if (c.spec.kind == 1) {
      for (int i = 0; i < c.spec.n; ++i) sse_chunk(c, i, "", true, "", false);
    } else if (!c.spec.echo_text.empty()) {
      sse_chunk(c, 0, c.spec.echo_text, false, "", false);
    }
  }

  std::string usage(const Call& c, int64_t gen) const {
    return "{\"prompt_tokens\":" + std::to_string(c.spec.prompt_tokens) + ",\"completion_tokens\":" + std::to_string(gen) +
           ",\"total_tokens\":" + std::to_string(c.spec.prompt_tokens + gen) + "}";
  }

  void emit(Call& c, int i, const std::string& piece) {
    if (piece.empty()) return;
    c.texts[i] += piece;
    if (c.spec.stream) sse_chunk(c, i, piece, false, "", false);
  }

  // returns true when the call is complete and can be forgotten
  bool handle(Call& c, const RespEvent& e) {
    const int i = e.seq_index;
    if (i < 0 || i >= c.spec.n) return false;
    if (e.aborted) {
      finish_call(c, true);
      return true;
    }
    if (c.spec.stream && !c.started) start_stream(c);
    if (e.token >= 0) {
      if (c.t_first == 0) {
        c.t_first = now_s();
        Metrics::instance().histogram_observe("time_to_first_token_latency_milliseconds", (c.t_first - c.spec.t_arrival) * 1e3);
      }
      c.ids[i].push_back(e.token);
      if (c.decoders[i] && c.finish[i].empty()) {
        bool stopped = false;
        emit(c, i, c.decoders[i]->push(e.token, &stopped));
        if (stopped) c.finish[i] = "stop";
      }
    }
    if (e.finished) {
      if (c.decoders[i] && c.finish[i].empty()) emit(c, i, c.decoders[i]->flush());
      if (c.finish[i].empty()) c.finish[i] = e.finish_reason.empty() ? "stop" : e.finish_reason;
      if (c.spec.stream) sse_chunk(c, i, "", false, c.finish[i], true);
    }
    if (e.request_finished) {
      finish_call(c, false);
      return true;
    }
    return false;
  }

  void finish_call(Call& c, bool aborted) {
    int64_t gen = 0;
    for (auto& v : c.ids) gen += (int64_t)v.size();
    const double now = now_s();
    Metrics& m = Metrics::instance();
    m.counter_add(aborted ? "server_request_total_fail" : "server_request_total_ok", 1.0);
    m.counter_add(aborted ? "request_status_total_cancelled" : "request_status_total_ok", 1.0);
    m.histogram_observe("num_generated_tokens_per_request", (double)gen);
    m.histogram_observe("num_prompt_tokens_per_request", (double)c.spec.prompt_tokens);
    m.counter_add("num_generated_tokens_total", (double)gen);
    m.counter_add("num_prompt_tokens_total", (double)c.spec.prompt_tokens);
    m.histogram_observe("end_2_end_latency_milliseconds", (now - c.spec.t_arrival) * 1e3);
    if (gen > 1 && c.t_first > 0)
      m.histogram_observe("inter_token_latency_milliseconds", (now - c.t_first) * 1e3 / (double)(gen - 1));
    if (!aborted) {
      if (c.spec.stream) {
        if (!c.started) start_stream(c);
        if (c.spec.include_usage) {
          std::string o = "data: " + head(c, c.spec.kind == 0 ? "text_completion" : "chat.completion.chunk");
          o += ",\"choices\":[],\"usage\":" + usage(c, gen) + "}\n\n";
          http_->stream_send(c.spec.http_id, o);
        }
        http_->stream_send(c.spec.http_id, "data: [DONE]\n\n");
        http_->stream_end(c.spec.http_id);
      } else {
        std::string o = head(c, c.spec.kind == 0 ? "text_completion" : "chat.completion");
        o += ",\"choices\":[";
        for (int i = 0; i < c.spec.n; ++i) {
          if (i) o += ",";
          o += "{\"index\":" + std::to_string(i);
          if (c.spec.kind == 0) {
            o += ",\"text\":";
            q(o, c.spec.echo_text + c.texts[i]);
          } else {
            o += ",\"message\":{\"role\":\"assistant\",\"content\":";
            q(o, c.texts[i]);
            o += "}";
          }
          o += ",\"finish_reason\":";
          q(o, c.finish[i].empty() ? std::string("stop") : c.finish[i]);
          if (c.spec.return_token_ids || !tok_) {
            o += ",\"token_ids\":[";
            for (size_t k = 0; k < c.ids[i].size(); ++k) {
              if (k) o += ",";
              o += std::to_string(c.ids[i][k]);
            }
            o += "]";
          }
          o += "}";
        }
        o += "],\"usage\":" + usage(c, gen) + "}";
        http_->respond(c.spec.http_id, 200, "application/json", o);
      }
    }
    RespDone d;
    d.request_id = c.spec.request_id;
    d.http_id = c.spec.http_id;
    d.generated = gen;
    d.prompt_tokens = c.spec.prompt_tokens;
    d.aborted = aborted;
    d.ttft_ms = c.t_first > 0 ? (c.t_first - c.spec.t_arrival) * 1e3 : 0;
    d.e2e_ms = (now - c.spec.t_arrival) * 1e3;
    std::lock_guard<std::mutex> lk(done_mu_);
    done_.push_back(std::move(d));
  }

  HttpServer* http_;
  std::shared_ptr<BpeTokenizer> tok_;
  std::vector<std::unique_ptr<Worker>> workers_;
  std::atomic<int64_t> next_handle_{1};
  std::atomic<int64_t> pending_{0}, processed_{0};
  std::atomic<bool> stopped_{false};
  std::mutex done_mu_;
  std::vector<RespDone> done_;
};

}  // namespace xllm
