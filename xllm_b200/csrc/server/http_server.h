// Epoll HTTP/1.1 server with chunked streaming (Server-Sent Events) for the OpenAI-compatible API.
//
// The reference serves HTTP through brpc (xllm/server/xllm_server.cpp:39-183, api_service/
// stream_call.h for SSE "progressive attachments"); brpc is not available here, so this is a
// self-contained transport: one epoll thread accepts connections, parses requests and writes
// responses; request handlers run elsewhere (the service loop polls `poll()` and answers through
// `respond()` / `stream_*()`), which keeps the engine loop single-threaded like the reference's
// scheduler thread.  A closed client socket is visible through `is_disconnected()` so that the
// service can abort the request (reference: call->is_disconnected(), continuous_scheduler.cpp:964).
#pragma once
#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace xllm {

struct HttpRequest {
  int64_t id = 0;
  std::string method, path, query, body;
  std::vector<std::pair<std::string, std::string>> headers;
  std::string header(const std::string& name) const {
    for (auto& h : headers)
      if (strcasecmp(h.first.c_str(), name.c_str()) == 0) return h.second;
    return std::string();
  }
};

class HttpServer {
 public:
  HttpServer() = default;
  ~HttpServer() { stop(); }

  // Returns the bound port (useful with port 0).  Throws on failure.
  int start(const std::string& host, int port) {
    listen_fd_ = ::socket(AF_INET, SOCK_STREAM | SOCK_NONBLOCK, 0);
    if (listen_fd_ < 0) throw std::runtime_error("socket() failed");
    int one = 1;
    setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)port);
    addr.sin_addr.s_addr = host.empty() || host == "0.0.0.0" ? INADDR_ANY : inet_addr(host.c_str());
    if (::bind(listen_fd_, (sockaddr*)&addr, sizeof(addr)) != 0 || ::listen(listen_fd_, 512) != 0) {
      ::close(listen_fd_);
      listen_fd_ = -1;
      throw std::runtime_error("cannot bind/listen on port " + std::to_string(port) + ": " + strerror(errno));
    }
    socklen_t len = sizeof(addr);
    getsockname(listen_fd_, (sockaddr*)&addr, &len);
    port_ = ntohs(addr.sin_port);
    epfd_ = epoll_create1(0);
    wake_fd_ = eventfd(0, EFD_NONBLOCK);
    add_fd(listen_fd_, EPOLLIN);
    add_fd(wake_fd_, EPOLLIN);
    running_ = true;
    thread_ = std::thread([this] { loop(); });
    return port_;
  }

  void stop() {
    if (!running_.exchange(false)) return;
    wake();
    if (thread_.joinable()) thread_.join();
    for (auto& kv : conns_) ::close(kv.first);
    conns_.clear();
    if (listen_fd_ >= 0) ::close(listen_fd_);
    if (epfd_ >= 0) ::close(epfd_);
    if (wake_fd_ >= 0) ::close(wake_fd_);
    listen_fd_ = epfd_ = wake_fd_ = -1;
  }
  int port() const { return port_; }

  // Requests received since the last call (waits up to timeout_ms for the first one).
  std::vector<HttpRequest> poll(int timeout_ms) {
    std::unique_lock<std::mutex> lk(mu_);
    if (inbox_.empty() && timeout_ms > 0)
      cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [this] { return !inbox_.empty() || !running_; });
    std::vector<HttpRequest> out(inbox_.begin(), inbox_.end());
    inbox_.clear();
    return out;
  }

  // Complete response with Content-Length.
  bool respond(int64_t id, int status, const std::string& content_type, const std::string& body,
               const std::vector<std::pair<std::string, std::string>>& extra_headers = {}) {
    std::string head = status_line(status) + "Content-Type: " + content_type + "\r\nContent-Length: " +
                       std::to_string(body.size()) + "\r\nConnection: keep-alive\r\n";
    for (auto& h : extra_headers) head += h.first + ": " + h.second + "\r\n";
    head += "\r\n";
    return enqueue(id, head + body, /*done=*/true);
  }
  // Streaming response: chunked transfer encoding (content_type "text/event-stream" for SSE).
  bool stream_begin(int64_t id, int status, const std::string& content_type) {
    return enqueue(id, status_line(status) + "Content-Type: " + content_type +
                           "\r\nCache-Control: no-cache\r\nTransfer-Encoding: chunked\r\nConnection: keep-alive\r\n\r\n",
                   false);
  }
  bool stream_send(int64_t id, const std::string& data) {
    if (data.empty()) return true;
    char len[32];
    snprintf(len, sizeof(len), "%zx\r\n", data.size());
    return enqueue(id, std::string(len) + data + "\r\n", false);
  }
  bool stream_end(int64_t id) { return enqueue(id, "0\r\n\r\n", true); }

  bool is_disconnected(int64_t id) {
    std::lock_guard<std::mutex> lk(mu_);
    return req_to_fd_.find(id) == req_to_fd_.end();
  }
  int64_t num_connections() {
    std::lock_guard<std::mutex> lk(mu_);
    return (int64_t)conns_.size();
  }

 private:
  struct Conn {
    std::string in;         // bytes received, not yet parsed
    std::string out;        // bytes to send
    int64_t active_req = 0; // request being answered (0: none)
    bool close_after = false;
  };

  static std::string status_line(int status) {
    const char* text = "OK";
    switch (status) {
      case 200: text = "OK"; break;
      case 400: text = "Bad Request"; break;
      case 404: text = "Not Found"; break;
      case 405: text = "Method Not Allowed"; break;
      case 413: text = "Payload Too Large"; break;
      case 429: text = "Too Many Requests"; break;
      case 500: text = "Internal Server Error"; break;
      case 503: text = "Service Unavailable"; break;
      default: text = "Status"; break;
    }
    return "HTTP/1.1 " + std::to_string(status) + " " + text + "\r\n";
  }
  void add_fd(int fd, uint32_t ev) {
    epoll_event e{};
    e.events = ev;
    e.data.fd = fd;
    epoll_ctl(epfd_, EPOLL_CTL_ADD, fd, &e);
  }
  void mod_fd(int fd, uint32_t ev) {
    epoll_event e{};
    e.events = ev;
    e.data.fd = fd;
    epoll_ctl(epfd_, EPOLL_CTL_MOD, fd, &e);
  }
  void wake() {
    uint64_t one = 1;
    ssize_t r = ::write(wake_fd_, &one, sizeof(one));
    (void)r;
  }

  bool enqueue(int64_t id, std::string data, bool done) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      auto it = req_to_fd_.find(id);
      if (it == req_to_fd_.end()) return false;
      outbox_.push_back({it->second, id, std::move(data), done});
    }
    wake();
    return true;
  }

  void close_conn(int fd) {
    epoll_ctl(epfd_, EPOLL_CTL_DEL, fd, nullptr);
    ::close(fd);
    std::lock_guard<std::mutex> lk(mu_);
    auto it = conns_.find(fd);
    if (it != conns_.end()) {
      if (it->second.active_req) req_to_fd_.erase(it->second.active_req);
      conns_.erase(it);
    }
  }

  // Full-string, range-checked decimal parse of a Content-Length value (no exceptions).
  static bool parse_length(const std::string& v, size_t* out) {
    size_t b = 0, e = v.size();
    while (b < e && (v[b] == ' ' || v[b] == '\t')) ++b;
    while (e > b && (v[e - 1] == ' ' || v[e - 1] == '\t' || v[e - 1] == '\r')) --e;
    if (b == e || e - b > 18) return false;
    size_t n = 0;
    for (size_t i = b; i < e; ++i) {
      if (v[i] < '0' || v[i] > '9') return false;
      n = n * 10 + (size_t)(v[i] - '0');
    }
    *out = n;
    return true;
  }

  // Answer `status` and close: the reply is queued, input is dropped from now on, and the caller
  // flushes (flush() closes the connection once the reply is out).  mu_ is held by the caller.
  void reject(Conn& c, int status) {
    c.out += status_line(status) + "Content-Length: 0\r\nConnection: close\r\n\r\n";
    c.close_after = true;
    c.in.clear();
  }

  // Parse as many complete requests as the buffer holds (one at a time per connection: the next
  // request of a keep-alive connection is parsed after the current one was answered).
  // Returns true when the connection has something to send (a rejection) and must be flushed.
  bool try_parse(int fd) {
    std::unique_lock<std::mutex> lk(mu_);
    auto it = conns_.find(fd);
    if (it == conns_.end()) return false;
    Conn& c = it->second;
    if (c.active_req != 0 || c.close_after) return false;
    const size_t he = c.in.find("\r\n\r\n");
    if (he == std::string::npos) {
      if (c.in.size() > (1u << 20)) { reject(c, 400); return true; }   // no end of headers within 1 MiB
      return false;
    }
    HttpRequest req;
    size_t line_end = c.in.find("\r\n");
    const std::string first = c.in.substr(0, line_end);
    const size_t s1 = first.find(' '), s2 = first.rfind(' ');
    if (s1 == std::string::npos || s2 == s1) { reject(c, 400); return true; }
    req.method = first.substr(0, s1);
    std::string target = first.substr(s1 + 1, s2 - s1 - 1);
    const size_t q = target.find('?');
    req.path = target.substr(0, q);
    if (q != std::string::npos) req.query = target.substr(q + 1);
    size_t pos = line_end + 2;
    size_t content_length = 0;
    while (pos < he) {
      const size_t e = c.in.find("\r\n", pos);
      const std::string line = c.in.substr(pos, e - pos);
      const size_t colon = line.find(':');
      if (colon != std::string::npos) {
        std::string k = line.substr(0, colon), v = line.substr(colon + 1);
        while (!v.empty() && v.front() == ' ') v.erase(0, 1);
        if (strcasecmp(k.c_str(), "content-length") == 0 && !parse_length(v, &content_length)) {
          reject(c, 400);
          return true;
        }
        req.headers.emplace_back(std::move(k), std::move(v));
      }
      pos = e + 2;
    }
    if (content_length > max_body_) { reject(c, 413); return true; }
    if (c.in.size() < he + 4 + content_length) return false;  // body still arriving
    req.body = c.in.substr(he + 4, content_length);
    c.in.erase(0, he + 4 + content_length);
    req.id = next_id_++;
    c.active_req = req.id;
    req_to_fd_[req.id] = fd;
    inbox_.push_back(std::move(req));
    lk.unlock();
    cv_.notify_all();
    return false;
  }

  void flush(int fd) {
    std::unique_lock<std::mutex> lk(mu_);
    auto it = conns_.find(fd);
    if (it == conns_.end()) return;
    Conn& c = it->second;
    while (!c.out.empty()) {
      const ssize_t n = ::send(fd, c.out.data(), c.out.size(), MSG_NOSIGNAL);
      if (n > 0) { c.out.erase(0, (size_t)n); continue; }
      if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) { mod_fd(fd, EPOLLIN | EPOLLOUT); return; }
      lk.unlock();
      close_conn(fd);
      return;
    }
    mod_fd(fd, EPOLLIN);
    if (c.close_after) {
      lk.unlock();
      close_conn(fd);
    }
  }

  void loop() {
    std::vector<epoll_event> evs(256);
    while (running_) {
      const int n = epoll_wait(epfd_, evs.data(), (int)evs.size(), 200);
      for (int i = 0; i < n; ++i) {
        const int fd = evs[i].data.fd;
        // nothing a single connection sends may end the serving thread: an exception raised while
        // its event is handled closes that connection only
        try {
          handle_event(fd, evs[i].events);
        } catch (...) {
          if (fd != listen_fd_ && fd != wake_fd_) close_conn(fd);
        }
      }
      drain_outbox();
    }
  }

  void handle_event(int fd, uint32_t events) {
    {
      {
        if (fd == listen_fd_) {
          while (true) {
            const int cfd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_NONBLOCK);
            if (cfd < 0) break;
            int one = 1;
            setsockopt(cfd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            { std::lock_guard<std::mutex> lk(mu_); conns_[cfd]; }
            add_fd(cfd, EPOLLIN);
          }
          return;
        }
        if (fd == wake_fd_) {
          uint64_t v;
          while (::read(wake_fd_, &v, sizeof(v)) > 0) {}
          return;
        }
        if (events & (EPOLLHUP | EPOLLERR)) { close_conn(fd); return; }
        if (events & EPOLLIN) {
          char buf[65536];
          bool closed = false;
          while (true) {
            const ssize_t r = ::recv(fd, buf, sizeof(buf), 0);
            if (r > 0) {
              std::lock_guard<std::mutex> lk(mu_);
              auto it = conns_.find(fd);
              // a connection that is being closed takes no more input (its buffer must not grow)
              if (it != conns_.end() && !it->second.close_after) it->second.in.append(buf, (size_t)r);
              continue;
            }
            if (r == 0) closed = true;
            else if (errno != EAGAIN && errno != EWOULDBLOCK) closed = true;
            break;
          }
          if (closed) { close_conn(fd); return; }
          if (try_parse(fd)) flush(fd);
        }
        if (events & EPOLLOUT) flush(fd);
      }
    }
  }

  // move queued responses into their connections
  void drain_outbox() {
    {
      std::vector<int> touched;
      {
        std::lock_guard<std::mutex> lk(mu_);
        for (auto& o : outbox_) {
          auto it = conns_.find(o.fd);
          if (it == conns_.end() || it->second.active_req != o.req) continue;
          it->second.out += o.data;
          if (o.done) {
            req_to_fd_.erase(o.req);
            it->second.active_req = 0;
          }
          touched.push_back(o.fd);
        }
        outbox_.clear();
      }
      for (int fd : touched) {
        flush(fd);
        if (try_parse(fd)) flush(fd);  // a pipelined request may already be buffered
      }
    }
  }

  struct Out {
    int fd;
    int64_t req;
    std::string data;
    bool done;
  };
  int listen_fd_ = -1, epfd_ = -1, wake_fd_ = -1, port_ = 0;
  std::atomic<bool> running_{false};
  std::thread thread_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::map<int, Conn> conns_;
  std::unordered_map<int64_t, int> req_to_fd_;
  std::deque<HttpRequest> inbox_;
  std::vector<Out> outbox_;
  int64_t next_id_ = 1;
  size_t max_body_ = 256u << 20;
};

}  // namespace xllm
