// Global proxy for xPyD serving: an HTTP/1.1 reverse proxy that runs every generation request in two phases,
// prefill on one instance and decode on another, choosing instances with the load balancers of lb.h.
//
//   client -> POST /v1/completions | /v1/chat/completions
//     1. X-Request-Id is added when absent                      (ngx_http_set_request_id_module.c:25)
//     2. the body is rewritten for prefill: max_tokens = 1, stream = false, stream_options removed, and sent to
//        a prefill instance                                      (ngx_http_prefill_module.c:515-651, 709-768)
//     3. the keys listed in --prefill-keys (default kv_transfer_params) are copied from the prefill response into
//        the original body; a prefill status >= 300 is passed through to the client        (:106-345)
//     4. the request goes to a decode instance; its response (SSE stream or JSON) is relayed as it arrives while
//        a body filter feeds token counters to the balancer      (pd_score...c:292-356, weighted_least_active...c:167-243)
//   Failed connects and 5xx answers eject the peer for --fail-timeout seconds and the request is retried on another
//   peer (nothing has reached the client at that point); when every attempt fails the last answer is passed through.
//   GET /health answers 200, GET /metrics lists per-peer load in Prometheus text format.
//
// Concurrency: an epoll accept loop feeds a pool of worker threads (blocking sockets with poll timeouts).  With
// --workers N the process forks N such workers sharing the listen socket and one MAP_SHARED block of balancer
// state, which gives the multi-worker semantics of the nginx shared-memory zones.
#include <arpa/inet.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <signal.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <queue>
#include <random>
#include <sstream>
#include <string>
#include <thread>
#include <unordered_set>
#include <vector>

#include "json_min.h"
#include "lb.h"

using namespace omni_proxy;

struct Endpoint { std::string host; int port; };
struct Config {
  std::string listen_host = "0.0.0.0";
  int listen_port = 8080;
  std::vector<Endpoint> prefill, decode;
  LbParams prefill_lb, decode_lb;
  std::vector<std::string> prefill_keys = {"kv_transfer_params"};
  int workers = 1, threads = 64, retries = 2;
  double timeout_s = 600.0, connect_timeout_s = 3.0;
  int log_level = 1;
  bool timeline = false;   // one "<<<Action" line per request stage on stderr, in the engine's format
  long long max_body_bytes = 64ll << 20;   // larger request bodies are refused with 413
};

static Config g_cfg;
static LbShared* g_shm_prefill = nullptr;
static LbShared* g_shm_decode = nullptr;
static LoadBalancer* g_lb_prefill = nullptr;
static LoadBalancer* g_lb_decode = nullptr;
static volatile sig_atomic_t g_stop = 0;

// Per-request timeline in the format of the engine's logger, so that one tool can merge the proxy's and the engines'
// lines by request id (wall clock: the processes share no monotonic origin).
static void timeline(const char* action, const std::string& rid) {
  if (!g_cfg.timeline) return;
  const double t = std::chrono::duration<double>(std::chrono::system_clock::now().time_since_epoch()).count();
  char line[512];
  const int n = snprintf(line, sizeof(line), "<<<Action: %s; Timestamp:%.6f; RequestID:%s; Role:proxy\n", action, t, rid.c_str());
  if (n > 0) (void)!write(STDERR_FILENO, line, (size_t)std::min<int>(n, (int)sizeof(line) - 1));   // one write: lines of concurrent requests do not interleave
}

static double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
#define LOG(level, ...) do { if (g_cfg.log_level >= level) { fprintf(stderr, "[omni_proxy] " __VA_ARGS__); fputc('\n', stderr); } } while (0)

// ------------------------------------------------------------------------------------------------ sockets
static bool wait_fd(int fd, short ev, double timeout_s) {
  struct pollfd p = {fd, ev, 0};
  int r = poll(&p, 1, (int)(timeout_s * 1000));
  return r > 0 && (p.revents & (ev | POLLHUP | POLLERR));
}
static bool send_all(int fd, const char* d, size_t n, double timeout_s) {
  size_t off = 0;
  while (off < n) {
    ssize_t w = send(fd, d + off, n - off, MSG_NOSIGNAL);
    if (w > 0) { off += (size_t)w; continue; }
    if (w < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) { if (!wait_fd(fd, POLLOUT, timeout_s)) return false; continue; }
    if (w < 0 && errno == EINTR) continue;
    return false;
  }
  return true;
}
static int connect_to(const Endpoint& ep, double timeout_s) {
  struct addrinfo hints = {}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(ep.host.c_str(), std::to_string(ep.port).c_str(), &hints, &res) != 0 || !res) return -1;
  int fd = socket(res->ai_family, SOCK_STREAM, 0);
  if (fd < 0) { freeaddrinfo(res); return -1; }
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  int rc = connect(fd, res->ai_addr, res->ai_addrlen);
  freeaddrinfo(res);
  if (rc < 0 && errno != EINPROGRESS) { close(fd); return -1; }
  if (rc < 0) {
    if (!wait_fd(fd, POLLOUT, timeout_s)) { close(fd); return -1; }
    int err = 0; socklen_t l = sizeof(err);
    getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &l);
    if (err) { close(fd); return -1; }
  }
  fcntl(fd, F_SETFL, fl);   // back to blocking; reads use poll for timeouts
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  return fd;
}

// ------------------------------------------------------------------------------------------------ HTTP
struct HttpMessage {
  std::string start_line;                                   // request line or status line
  std::vector<std::pair<std::string, std::string>> headers;
  std::string body;
  int status = 0;
  std::string method, path;
  std::string header(const std::string& name) const {
    for (auto& h : headers) if (strcasecmp(h.first.c_str(), name.c_str()) == 0) return h.second;
    return "";
  }
  void set_header(const std::string& name, const std::string& v) {
    for (auto& h : headers) if (strcasecmp(h.first.c_str(), name.c_str()) == 0) { h.second = v; return; }
    headers.push_back({name, v});
  }
  void remove_header(const std::string& name) {
    for (size_t i = 0; i < headers.size();)
      if (strcasecmp(headers[i].first.c_str(), name.c_str()) == 0) headers.erase(headers.begin() + i); else ++i;
  }
  std::string serialize_head() const {
    std::string s = start_line + "\r\n";
    for (auto& h : headers) s += h.first + ": " + h.second + "\r\n";
    return s + "\r\n";
  }
};

// reads until the end of the header block; `rest` receives bytes read past it
static bool read_head(int fd, HttpMessage& m, std::string& rest, double timeout_s) {
  std::string buf = rest;
  rest.clear();
  size_t pos;
  char tmp[8192];
  while ((pos = buf.find("\r\n\r\n")) == std::string::npos) {
    if (buf.size() > (1u << 20)) return false;
    if (!wait_fd(fd, POLLIN, timeout_s)) return false;
    ssize_t r = recv(fd, tmp, sizeof(tmp), 0);
    if (r <= 0) return false;
    buf.append(tmp, (size_t)r);
  }
  rest = buf.substr(pos + 4);
  std::istringstream in(buf.substr(0, pos));
  std::string line;
  if (!std::getline(in, line)) return false;
  if (!line.empty() && line.back() == '\r') line.pop_back();
  m.start_line = line;
  if (line.compare(0, 5, "HTTP/") == 0) {
    size_t sp = line.find(' ');
    m.status = sp == std::string::npos ? 0 : atoi(line.c_str() + sp + 1);
  } else {
    std::istringstream ls(line);
    ls >> m.method >> m.path;
  }
  while (std::getline(in, line)) {
    if (!line.empty() && line.back() == '\r') line.pop_back();
    size_t c = line.find(':');
    if (c == std::string::npos) continue;
    size_t v = c + 1;
    while (v < line.size() && line[v] == ' ') ++v;
    m.headers.push_back({line.substr(0, c), line.substr(v)});
  }
  return true;
}

static bool read_exact(int fd, std::string& out, size_t n, std::string& rest, double timeout_s) {
  out = rest.substr(0, std::min(n, rest.size()));
  rest.erase(0, out.size());
  char tmp[16384];
  while (out.size() < n) {
    if (!wait_fd(fd, POLLIN, timeout_s)) return false;
    ssize_t r = recv(fd, tmp, std::min(sizeof(tmp), n - out.size()), 0);
    if (r <= 0) return false;
    out.append(tmp, (size_t)r);
  }
  return true;
}

// whole body of a response (Content-Length, chunked, or until close)
static bool read_body_all(int fd, HttpMessage& m, std::string& rest, double timeout_s) {
  const std::string cl = m.header("Content-Length");
  if (!cl.empty()) return read_exact(fd, m.body, (size_t)atoll(cl.c_str()), rest, timeout_s);
  const bool chunked = strcasecmp(m.header("Transfer-Encoding").c_str(), "chunked") == 0;
  std::string raw = rest;
  rest.clear();
  char tmp[16384];
  while (true) {
    if (chunked) {   // try to decode what we have
      std::string body;
      size_t i = 0;
      bool done = false, need_more = false;
      while (true) {
        size_t e = raw.find("\r\n", i);
        if (e == std::string::npos) { need_more = true; break; }
        const size_t len = strtoul(raw.c_str() + i, nullptr, 16);
        if (len == 0) { done = true; break; }
        if (raw.size() < e + 2 + len + 2) { need_more = true; break; }
        body.append(raw, e + 2, len);
        i = e + 2 + len + 2;
      }
      if (done) { m.body = body; return true; }
      (void)need_more;
    }
    if (!wait_fd(fd, POLLIN, timeout_s)) return !chunked && !raw.empty() ? (m.body = raw, true) : false;
    ssize_t r = recv(fd, tmp, sizeof(tmp), 0);
    if (r < 0) return false;
    if (r == 0) { if (chunked) return false; m.body = raw; return true; }
    raw.append(tmp, (size_t)r);
  }
}

static void send_simple(int fd, int status, const std::string& reason, const std::string& body,
                        const std::string& ctype = "application/json") {
  std::string s = "HTTP/1.1 " + std::to_string(status) + " " + reason + "\r\nContent-Type: " + ctype +
                  "\r\nContent-Length: " + std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n" + body;
  send_all(fd, s.data(), s.size(), 10.0);
}

static std::string make_request_id() {
  static thread_local std::mt19937_64 rng(std::random_device{}());
  char b[40];
  uint64_t a = rng(), c = rng();
  snprintf(b, sizeof(b), "%08x-%04x-4%03x-%04x-%012llx", (unsigned)(a >> 32), (unsigned)(a >> 16) & 0xffff,
           (unsigned)a & 0xfff, (unsigned)((c >> 48) & 0x3fff) | 0x8000, (unsigned long long)(c & 0xffffffffffffULL));
  return b;
}

// ------------------------------------------------------------------------------------------------ PD flow
static std::string build_prefill_body(const std::string& body) {
  std::string b = body;
  json_set(b, "max_tokens", "1");
  json_set(b, "stream", "false");
  json_remove(b, "stream_options");
  return b;
}

// returns true and fills `out` (full response) when some prefill peer answered
static bool run_prefill(const HttpMessage& req, const std::string& body, HttpMessage& out) {
  const int64_t len = (int64_t)req.body.size();
  g_lb_decode->prefill_started(len);
  bool ok = false, have_error_response = false;
  for (int attempt = 0; attempt <= g_cfg.retries && !ok; ++attempt) {
    Ticket t = g_lb_prefill->get_peer(len, now_s());
    int up = connect_to(g_cfg.prefill[t.peer], g_cfg.connect_timeout_s);
    if (up < 0) {
      LOG(1, "prefill peer %d unreachable", t.peer);
      g_lb_prefill->free_peer(t, true, now_s());
      continue;
    }
    HttpMessage r = req;
    r.set_header("Content-Length", std::to_string(body.size()));
    r.set_header("Connection", "close");
    r.remove_header("Transfer-Encoding");
    std::string wire = r.serialize_head() + body;
    std::string rest;
    HttpMessage resp;
    timeline("Proxy sends to prefill", req.header("X-Request-Id"));
    const bool got = send_all(up, wire.data(), wire.size(), g_cfg.timeout_s) && read_head(up, resp, rest, g_cfg.timeout_s) &&
                     read_body_all(up, resp, rest, g_cfg.timeout_s);
    close(up);
    if (got) timeline("Proxy got prefill response", req.header("X-Request-Id"));
    // An instance that answers 5xx is reachable but not serving (its engine fails, it is out of memory): that counts
    // against it like a refused connection, and the request, which has produced nothing yet, goes to another peer.
    // If every attempt ends that way the last answer is passed through to the client.
    const bool server_error = got && resp.status >= 500;
    g_lb_prefill->free_peer(t, !got || server_error, now_s());
    if (server_error) {
      LOG(1, "prefill peer %d answered %d", t.peer, resp.status);
      out = resp;
      have_error_response = true;
      continue;
    }
    if (got) { out = resp; ok = true; }
  }
  g_lb_decode->prefill_finished(len);
  return ok || have_error_response;
}

// ------------------------------------------------------------------------------------------------ stream relay
// Once a decode instance has started to answer, the rest of the (possibly minutes-long) token stream is moved by one
// event loop instead of the worker thread that set the request up: thousands of open streams then cost a file
// descriptor pair each, not a thread each, as in the event-driven proxy of the reference.  The loop forwards bytes
// upstream -> client, runs the body filters (token counters for the balancers) on what passes, and gives the peer
// back when the upstream closes.  A client that reads slowly only stalls its own stream: its bytes wait in a pending
// buffer and its upstream is not read until the buffer has drained.
struct RelayConn;
struct RelayTag { RelayConn* c; bool is_client; };
struct RelayConn {
  int up = -1, client = -1;
  Ticket t;
  std::string rid, tail, pending;
  bool reading = true;
  bool server_error = false;  // the upstream answered 5xx: relayed, but counted against the peer
  double last_activity = 0;   // monotonic seconds of the last byte moved in either direction
  RelayTag up_tag{this, false}, client_tag{this, true};   // what the event loop gets back from epoll
};

static void scan_counters(RelayConn& c, const char* buf, size_t n) {
  std::string view = c.tail + std::string(buf, n);
  long long v, pn, on;
  if (find_int_after(view, "total_tokens", v)) g_lb_decode->on_decoded_tokens(c.t, v);
  if (find_int_after(view, "output_num_token", on)) {
    pn = 0;
    find_int_after(view, "prompt_num_token", pn);
    g_lb_decode->on_token_counts(c.t, pn, on);
  }
  c.tail = view.size() > 64 ? view.substr(view.size() - 64) : view;
}

class Relay {
 public:
  Relay() {
    ep_ = epoll_create1(0);
    wake_ = eventfd(0, EFD_NONBLOCK);
    struct epoll_event ev = {};
    ev.events = EPOLLIN;
    ev.data.ptr = nullptr;       // the wake-up descriptor
    epoll_ctl(ep_, EPOLL_CTL_ADD, wake_, &ev);
    th_ = std::thread([this] { loop(); });
  }
  ~Relay() { stop(); }
  void stop() {
    if (stopped_.exchange(true)) return;
    uint64_t one = 1;
    (void)!write(wake_, &one, sizeof(one));
    if (th_.joinable()) th_.join();
    for (auto* c : conns_) finish(c, false);
    conns_.clear();
    for (auto* c : incoming_) { n_open_++; finish(c, false); }   // handed over but never armed
    incoming_.clear();
    close(ep_);
    close(wake_);
  }
  // takes ownership of both descriptors and of the ticket
  void add(RelayConn* c) {
    fcntl(c->up, F_SETFL, fcntl(c->up, F_GETFL, 0) | O_NONBLOCK);
    fcntl(c->client, F_SETFL, fcntl(c->client, F_GETFL, 0) | O_NONBLOCK);
    { std::lock_guard<std::mutex> lk(mu_); incoming_.push_back(c); }
    uint64_t one = 1;
    (void)!write(wake_, &one, sizeof(one));
  }
  size_t open_streams() const { return n_open_.load(); }

 private:
  using Tag = RelayTag;
  void arm(RelayConn* c) {
    struct epoll_event ev = {};
    ev.events = EPOLLIN;
    ev.data.ptr = &c->up_tag;
    epoll_ctl(ep_, EPOLL_CTL_ADD, c->up, &ev);
    struct epoll_event ec = {};
    ec.events = 0;
    ec.data.ptr = &c->client_tag;
    epoll_ctl(ep_, EPOLL_CTL_ADD, c->client, &ec);
  }
  // which events are wanted depends on whether bytes are waiting for the client
  void want(RelayConn* c) {
    struct epoll_event ev = {};
    ev.data.ptr = &c->up_tag;
    ev.events = (c->pending.empty() && c->reading) ? EPOLLIN : 0;
    epoll_ctl(ep_, EPOLL_CTL_MOD, c->up, &ev);
    struct epoll_event ec = {};
    ec.data.ptr = &c->client_tag;
    ec.events = c->pending.empty() ? 0 : EPOLLOUT;
    epoll_ctl(ep_, EPOLL_CTL_MOD, c->client, &ec);
  }
  void finish(RelayConn* c, bool failed) {
    epoll_ctl(ep_, EPOLL_CTL_DEL, c->up, nullptr);
    epoll_ctl(ep_, EPOLL_CTL_DEL, c->client, nullptr);
    close(c->up);
    shutdown(c->client, SHUT_RDWR);
    close(c->client);
    g_lb_decode->free_peer(c->t, failed || c->server_error, now_s());
    timeline("Proxy finished request", c->rid);
    n_open_--;
    delete c;
  }
  // true while the connection lives
  bool flush(RelayConn* c) {
    while (!c->pending.empty()) {
      ssize_t w = send(c->client, c->pending.data(), c->pending.size(), MSG_NOSIGNAL);
      if (w > 0) { c->pending.erase(0, (size_t)w); continue; }
      if (w < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) return true;
      if (w < 0 && errno == EINTR) continue;
      return false;     // the client went away
    }
    return true;
  }
  void loop() {
    char buf[32768];
    std::vector<struct epoll_event> evs(256);
    while (!stopped_) {
      int n = epoll_wait(ep_, evs.data(), (int)evs.size(), 500);
      {
        std::lock_guard<std::mutex> lk(mu_);
        for (auto* c : incoming_) { c->last_activity = now_s(); conns_.insert(c); n_open_++; arm(c); }
        incoming_.clear();
      }
      std::vector<RelayConn*> dead;
      auto is_dead = [&](RelayConn* c) { return std::find(dead.begin(), dead.end(), c) != dead.end(); };
      for (int i = 0; i < n; ++i) {
        Tag* tag = (Tag*)evs[i].data.ptr;
        if (tag == nullptr) { uint64_t v; (void)!read(wake_, &v, sizeof(v)); continue; }
        RelayConn* c = tag->c;
        if (is_dead(c)) continue;
        c->last_activity = now_s();
        if (tag->is_client) {
          if (!flush(c)) { dead.push_back(c); continue; }
          if (c->pending.empty()) {
            if (!c->reading) { dead.push_back(c); continue; }   // upstream had closed: these were the last bytes
            want(c);
          }
          continue;
        }
        bool closed = false, lost_client = false;
        while (c->pending.empty()) {
          ssize_t r = recv(c->up, buf, sizeof(buf), 0);
          if (r > 0) {
            scan_counters(*c, buf, (size_t)r);
            c->pending.assign(buf, (size_t)r);
            if (!flush(c)) { lost_client = true; break; }
            continue;
          }
          if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) break;
          if (r < 0 && errno == EINTR) continue;
          closed = true;      // end of the stream (or an upstream error)
          break;
        }
        if (lost_client || (closed && c->pending.empty())) { dead.push_back(c); continue; }
        if (closed) c->reading = false;
        want(c);
      }
      for (auto* c : dead) {
        conns_.erase(c);
        finish(c, false);
      }
      // a stream on which nothing has moved for the upstream time-out is given up (its peer counts a failure)
      const double now = now_s();
      if (now - last_sweep_ > 1.0) {
        last_sweep_ = now;
        std::vector<RelayConn*> idle;
        for (auto* c : conns_) if (now - c->last_activity > g_cfg.timeout_s) idle.push_back(c);
        for (auto* c : idle) {
          LOG(1, "stream %s idle for %.0f s: closed", c->rid.c_str(), now - c->last_activity);
          conns_.erase(c);
          finish(c, true);
        }
      }
    }
  }
  int ep_ = -1, wake_ = -1;
  std::thread th_;
  std::mutex mu_;
  std::vector<RelayConn*> incoming_;
  std::unordered_set<RelayConn*> conns_;
  std::atomic<bool> stopped_{false};
  std::atomic<size_t> n_open_{0};
  double last_sweep_ = 0;
};
static Relay* g_relay = nullptr;

// relays the decode response to the client as it arrives; returns false when the client went away
static bool run_decode(int client, const HttpMessage& req, const std::string& body, bool& handed_over) {
  const int64_t len = (int64_t)req.body.size();
  handed_over = false;
  for (int attempt = 0; attempt <= g_cfg.retries; ++attempt) {
    Ticket t = g_lb_decode->get_peer(len, now_s());
    int up = connect_to(g_cfg.decode[t.peer], g_cfg.connect_timeout_s);
    if (up < 0) {
      LOG(1, "decode peer %d unreachable", t.peer);
      g_lb_decode->free_peer(t, true, now_s());
      continue;
    }
    HttpMessage r = req;
    r.set_header("Content-Length", std::to_string(body.size()));
    r.set_header("Connection", "close");
    r.remove_header("Transfer-Encoding");
    std::string wire = r.serialize_head() + body;
    timeline("Proxy sends to decode", req.header("X-Request-Id"));
    bool sent = send_all(up, wire.data(), wire.size(), g_cfg.timeout_s);
    // the first bytes are awaited here, so that a peer that accepts the connection and then dies is still retried on
    // another one; everything after them belongs to the relay loop
    char buf[16384];
    ssize_t n = -1;
    if (sent && wait_fd(up, POLLIN, g_cfg.timeout_s)) n = recv(up, buf, sizeof(buf), 0);
    if (n <= 0) {
      close(up);
      g_lb_decode->free_peer(t, true, now_s());
      continue;
    }
    // "HTTP/1.1 5xx": the instance is up but cannot serve.  Nothing has been sent to the client yet, so another
    // instance gets the request; the last attempt's answer is relayed as it is.  Either way it counts as a failure.
    const bool server_error = n >= 12 && memcmp(buf, "HTTP/1.", 7) == 0 && buf[8] == ' ' && buf[9] == '5';
    if (server_error && attempt < g_cfg.retries) {
      LOG(1, "decode peer %d answered 5xx", t.peer);
      close(up);
      g_lb_decode->free_peer(t, true, now_s());
      continue;
    }
    timeline("Proxy relays first decode bytes", req.header("X-Request-Id"));
    RelayConn* c = new RelayConn();
    c->up = up; c->client = client; c->t = t; c->rid = req.header("X-Request-Id");
    c->server_error = server_error;
    scan_counters(*c, buf, (size_t)n);
    if (!send_all(client, buf, (size_t)n, g_cfg.timeout_s)) {   // the client is already gone
      close(up);
      g_lb_decode->free_peer(c->t, false, now_s());
      delete c;
      return false;
    }
    g_relay->add(c);
    handed_over = true;
    return true;
  }
  send_simple(client, 502, "Bad Gateway", "{\"error\":\"no decode instance reachable\"}");
  return true;
}

static std::string metrics_text() {
  std::ostringstream o;
  if (g_relay) o << "omni_proxy_open_streams " << g_relay->open_streams() << "\n";
  auto dump = [&](const char* pool, LoadBalancer* lb) {
    if (!lb) return;
    for (int i = 0; i < lb->n_peers(); ++i) {
      const PeerState p = lb->peer(i);
      o << "omni_proxy_active_requests{pool=\"" << pool << "\",peer=\"" << i << "\"} " << p.active_requests << "\n";
      o << "omni_proxy_request_length{pool=\"" << pool << "\",peer=\"" << i << "\"} " << p.total_request_length << "\n";
      o << "omni_proxy_decode_tokens{pool=\"" << pool << "\",peer=\"" << i << "\"} " << p.total_decode_num << "\n";
      o << "omni_proxy_served_total{pool=\"" << pool << "\",peer=\"" << i << "\"} " << p.served << "\n";
      o << "omni_proxy_peer_up{pool=\"" << pool << "\",peer=\"" << i << "\"} " << (lb->is_up(i, now_s()) ? 1 : 0) << "\n";
    }
  };
  dump("prefill", g_lb_prefill);
  dump("decode", g_lb_decode);
  return o.str();
}

static void handle_connection(int client) {
  std::string rest;
  HttpMessage req;
  if (!read_head(client, req, rest, 30.0)) { close(client); return; }
  const std::string cl = req.header("Content-Length");
  if (!cl.empty()) {
    // the length is the client's claim: refuse what is not a number or more than a request can reasonably be, instead
    // of buffering whatever arrives
    char* end = nullptr;
    errno = 0;
    const long long n = strtoll(cl.c_str(), &end, 10);
    if (end == cl.c_str() || *end != '\0' || errno != 0 || n < 0) {
      send_simple(client, 400, "Bad Request", "{\"error\":\"invalid Content-Length\"}");
      close(client);
      return;
    }
    if (n > g_cfg.max_body_bytes) {
      send_simple(client, 413, "Payload Too Large", "{\"error\":\"request body too large\"}");
      close(client);
      return;
    }
    if (!read_exact(client, req.body, (size_t)n, rest, 60.0)) { close(client); return; }
  } else if (strcasecmp(req.header("Transfer-Encoding").c_str(), "chunked") == 0) {
    // a chunked request body is put together here and forwarded with a Content-Length
    if (!read_body_all(client, req, rest, 60.0) || (long long)req.body.size() > g_cfg.max_body_bytes) {
      send_simple(client, 400, "Bad Request", "{\"error\":\"unreadable chunked body\"}");
      close(client);
      return;
    }
    req.remove_header("Transfer-Encoding");
  }
  if (req.method.empty() || req.path.empty() || req.path[0] != '/') {
    send_simple(client, 400, "Bad Request", "{\"error\":\"malformed request line\"}");
    close(client);
    return;
  }
  if (req.method == "GET" && req.path == "/health") { send_simple(client, 200, "OK", "{\"status\":\"ok\"}"); close(client); return; }
  if (req.method == "GET" && req.path == "/metrics") { send_simple(client, 200, "OK", metrics_text(), "text/plain; version=0.0.4"); close(client); return; }
  if (req.header("X-Request-Id").empty()) req.set_header("X-Request-Id", make_request_id());
  const std::string rid = req.header("X-Request-Id");
  timeline("Proxy got request", rid);
  std::string body = req.body;
  const bool generation = req.method == "POST" && (req.path == "/v1/completions" || req.path == "/v1/chat/completions");
  if (generation && !g_cfg.prefill.empty()) {
    HttpMessage presp;
    if (!run_prefill(req, build_prefill_body(req.body), presp)) {
      send_simple(client, 502, "Bad Gateway", "{\"error\":\"no prefill instance reachable\"}");
      close(client);
      return;
    }
    if (presp.status >= 300) {   // pass the prefill failure through unchanged
      presp.set_header("Content-Length", std::to_string(presp.body.size()));
      presp.remove_header("Transfer-Encoding");
      presp.set_header("Connection", "close");
      std::string wire = presp.serialize_head() + presp.body;
      send_all(client, wire.data(), wire.size(), 30.0);
      close(client);
      return;
    }
    for (const auto& key : g_cfg.prefill_keys) {
      std::string v;
      if (json_get(presp.body, key, v)) json_set(body, key, v);
    }
  }
  bool handed_over = false;
  run_decode(client, req, body, handed_over);
  if (handed_over) return;          // the relay loop owns the descriptors now and closes them at the end of the stream
  timeline("Proxy finished request", rid);
  shutdown(client, SHUT_RDWR);
  close(client);
}

// ------------------------------------------------------------------------------------------------ server
class Pool {
 public:
  explicit Pool(int n) {
    for (int i = 0; i < n; ++i) ts_.emplace_back([this] { run(); });
  }
  void push(int fd) {
    { std::lock_guard<std::mutex> lk(mu_); q_.push(fd); }
    cv_.notify_one();
  }
  void stop() {
    { std::lock_guard<std::mutex> lk(mu_); stop_ = true; }
    cv_.notify_all();
    for (auto& t : ts_) t.join();
  }
 private:
  void run() {
    while (true) {
      int fd;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return stop_ || !q_.empty(); });
        if (stop_ && q_.empty()) return;
        fd = q_.front();
        q_.pop();
      }
      handle_connection(fd);
    }
  }
  std::vector<std::thread> ts_;
  std::queue<int> q_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool stop_ = false;
};

static void serve(int lfd) {
  Relay relay;            // per worker process
  g_relay = &relay;
  Pool pool(g_cfg.threads);
  int ep = epoll_create1(0);
  struct epoll_event ev = {};
  ev.events = EPOLLIN;
  ev.data.fd = lfd;
  epoll_ctl(ep, EPOLL_CTL_ADD, lfd, &ev);
  while (!g_stop) {
    struct epoll_event out[16];
    int n = epoll_wait(ep, out, 16, 200);
    for (int i = 0; i < n; ++i) {
      while (true) {
        int c = accept(lfd, nullptr, nullptr);
        if (c < 0) break;
        int one = 1;
        setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        pool.push(c);
      }
    }
  }
  pool.stop();
  relay.stop();
  g_relay = nullptr;
  close(ep);
}

static std::vector<Endpoint> parse_endpoints(const std::string& s) {
  std::vector<Endpoint> out;
  std::istringstream in(s);
  std::string item;
  while (std::getline(in, item, ',')) {
    if (item.empty()) continue;
    size_t c = item.rfind(':');
    if (c == std::string::npos) continue;
    out.push_back({item.substr(0, c), atoi(item.c_str() + c + 1)});
  }
  return out;
}

static void on_signal(int) { g_stop = 1; }

static LbShared* alloc_shared() {
  void* p = mmap(nullptr, sizeof(LbShared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
  if (p == MAP_FAILED) { perror("mmap"); exit(1); }
  memset(p, 0, sizeof(LbShared));
  return (LbShared*)p;
}

int main(int argc, char** argv) {
  bool dump = false;
  std::string p_policy = "pd_score_balance", d_policy = "pd_score_balance";
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto val = [&]() -> std::string { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--listen") { std::string v = val(); size_t c = v.rfind(':'); if (c != std::string::npos) { g_cfg.listen_host = v.substr(0, c); g_cfg.listen_port = atoi(v.c_str() + c + 1); } else g_cfg.listen_port = atoi(v.c_str()); }
    else if (a == "--prefill-servers" || a == "--prefill-servers-list") g_cfg.prefill = parse_endpoints(val());
    else if (a == "--decode-servers" || a == "--decode-servers-list") g_cfg.decode = parse_endpoints(val());
    else if (a == "--prefill-lb" || a == "--prefill-lb-sdk") p_policy = val();
    else if (a == "--decode-lb" || a == "--decode-lb-sdk") d_policy = val();
    else if (a == "--prefill-keys") { g_cfg.prefill_keys.clear(); std::istringstream in(val()); std::string k; while (std::getline(in, k, ',')) if (!k.empty()) g_cfg.prefill_keys.push_back(k); }
    else if (a == "--decode-req-limit") g_cfg.decode_lb.decode_req_limit = atoi(val().c_str());
    else if (a == "--batch-size") { int b = atoi(val().c_str()); g_cfg.decode_lb.batch_size = b; g_cfg.prefill_lb.batch_size = b; }
    else if (a == "--req-len-weight") g_cfg.decode_lb.req_len_weight = g_cfg.prefill_lb.req_len_weight = atof(val().c_str());
    else if (a == "--decay-factor") g_cfg.decode_lb.decay_factor = g_cfg.prefill_lb.decay_factor = atof(val().c_str());
    else if (a == "--greedy-warmup") g_cfg.prefill_lb.warmup = g_cfg.decode_lb.warmup = atof(val().c_str());
    else if (a == "--greedy-exp") g_cfg.prefill_lb.exponent = g_cfg.decode_lb.exponent = atof(val().c_str());
    else if (a == "--fail-timeout") g_cfg.prefill_lb.fail_timeout_s = g_cfg.decode_lb.fail_timeout_s = atof(val().c_str());
    else if (a == "--workers") g_cfg.workers = std::max(1, atoi(val().c_str()));
    else if (a == "--threads") g_cfg.threads = std::max(1, atoi(val().c_str()));
    else if (a == "--retries") g_cfg.retries = atoi(val().c_str());
    else if (a == "--max-body-mb") g_cfg.max_body_bytes = (long long)(atof(val().c_str()) * (1 << 20));
    else if (a == "--timeout") g_cfg.timeout_s = atof(val().c_str());
    else if (a == "--log-level") g_cfg.log_level = atoi(val().c_str());
    else if (a == "--timeline") g_cfg.timeline = true;
    else if (a == "--dump-config") dump = true;
    else if (a == "--help") { printf("omni_proxy --listen host:port --prefill-servers h:p,... --decode-servers h:p,... [--prefill-lb P] [--decode-lb P]\n  policies: pd_score_balance prefill_score_balance weighted_least_active length_balance greedy_timeout auto_balance_controller least_total_load round_robin\n"); return 0; }
    else { fprintf(stderr, "unknown option %s\n", a.c_str()); return 2; }
  }
  g_cfg.prefill_lb.policy = p_policy == "pd_score_balance" ? "pd_score_balance_prefill" : p_policy;
  g_cfg.decode_lb.policy = d_policy == "pd_score_balance" ? "pd_score_balance_decode" : d_policy;
  if (dump) {
    printf("{\"listen\":\"%s:%d\",\"prefill\":%zu,\"decode\":%zu,\"prefill_lb\":\"%s\",\"decode_lb\":\"%s\",\"workers\":%d,\"threads\":%d}\n",
           g_cfg.listen_host.c_str(), g_cfg.listen_port, g_cfg.prefill.size(), g_cfg.decode.size(),
           g_cfg.prefill_lb.policy.c_str(), g_cfg.decode_lb.policy.c_str(), g_cfg.workers, g_cfg.threads);
    return 0;
  }
  if (g_cfg.decode.empty()) { fprintf(stderr, "--decode-servers is required\n"); return 2; }
  signal(SIGPIPE, SIG_IGN);
  signal(SIGINT, on_signal);
  signal(SIGTERM, on_signal);
  g_shm_prefill = alloc_shared();
  g_shm_decode = alloc_shared();
  if (!g_cfg.prefill.empty()) g_lb_prefill = new LoadBalancer(g_shm_prefill, (int)g_cfg.prefill.size(), g_cfg.prefill_lb);
  g_lb_decode = new LoadBalancer(g_shm_decode, (int)g_cfg.decode.size(), g_cfg.decode_lb);

  int lfd = socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  struct sockaddr_in addr = {};
  addr.sin_family = AF_INET;
  addr.sin_port = htons((uint16_t)g_cfg.listen_port);
  addr.sin_addr.s_addr = g_cfg.listen_host == "0.0.0.0" ? INADDR_ANY : inet_addr(g_cfg.listen_host.c_str());
  if (bind(lfd, (struct sockaddr*)&addr, sizeof(addr)) < 0 || listen(lfd, 1024) < 0) { perror("bind/listen"); return 1; }
  fcntl(lfd, F_SETFL, fcntl(lfd, F_GETFL, 0) | O_NONBLOCK);
  LOG(1, "listening on %s:%d, %zu prefill / %zu decode peers, lb %s / %s", g_cfg.listen_host.c_str(), g_cfg.listen_port,
      g_cfg.prefill.size(), g_cfg.decode.size(), g_cfg.prefill_lb.policy.c_str(), g_cfg.decode_lb.policy.c_str());
  std::vector<pid_t> kids;
  for (int w = 1; w < g_cfg.workers; ++w) {
    pid_t pid = fork();
    if (pid == 0) { serve(lfd); _exit(0); }
    kids.push_back(pid);
  }
  serve(lfd);
  for (pid_t k : kids) { kill(k, SIGTERM); waitpid(k, nullptr, 0); }
  close(lfd);
  return 0;
}
