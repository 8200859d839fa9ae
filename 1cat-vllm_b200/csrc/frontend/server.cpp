// Native front end: an HTTP/1.1 server (epoll, one thread) with its own tokenizer that drives an engine-core process over the
// engine's ZMQ + msgpack protocol — the same sockets, handshake and frames the Python clients use (engine/core_proc.py):
//   ROUTER (bound here)  <- DEALER of the engine: frames [identity, kind, msgpack body]; kind 0 = add request, 1 = abort
//   PULL   (bound here)  <- PUSH of the engine:   frame 0 = msgpack {"outputs": [{request_id, new_token_ids, finish_reason, ...}]}
// Routes: GET /health, GET /v1/models, POST /tokenize, POST /detokenize, POST /v1/completions (text or token-id prompts, server-sent
// events when "stream" is true). A second thread blocks on the PULL socket and hands deltas to the HTTP thread through a queue and an
// eventfd; each socket is used by one thread only. A client that disconnects aborts its request in the engine.
// The engine is started by this program (--engine-cmd, with {input} and {output} replaced by the socket addresses) or attaches to
// the addresses given with --input-addr / --output-addr.
// (reference: rust/src/server (HTTP front end), rust/src/engine-core-client (ZMQ/msgpack client), rust/src/tokenizer)
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <deque>
#include <map>
#include <mutex>
#include <thread>

#include "tokenizer.h"
#include "value.h"
#include "zmq_dyn.h"

using namespace fe;

namespace {

struct Delta {
  std::string request_id;
  std::vector<int> tokens;
  int finish = -1;  // FinishReason of the engine: 0 stop, 1 length, 2 abort, 3 error; -1 = still running
  std::string stop_reason;
};

struct Conn {
  int fd = -1;
  std::string in, out;
  std::string active_request;  // id of the completion this connection is waiting for
  bool close_after = false;
};

struct Pending {
  int fd = -1;
  bool stream = false, echo_ids = false;
  int n_prompt = 0;
  std::vector<int> ids;
  std::string text, held;  // decoded text so far; bytes of an unfinished UTF-8 sequence
  long created = 0;
};

std::atomic<bool> g_stop{false};
void on_signal(int) { g_stop = true; }

size_t utf8_complete_prefix(const std::string& s) {  // bytes of s that form whole code points
  size_t n = s.size(), i = n;
  int back = 0;
  while (i > 0 && back < 4) {
    unsigned char c = (unsigned char)s[i - 1];
    if ((c & 0xC0) != 0x80) {
      int need = c >= 0xF0 ? 4 : c >= 0xE0 ? 3 : c >= 0xC0 ? 2 : 1;
      return (n - (i - 1) >= (size_t)need) ? n : i - 1;
    }
    --i;
    ++back;
  }
  return n;
}

class Server {
 public:
  Tokenizer tok;
  Zmq z;
  void *ctx = nullptr, *router = nullptr, *pull = nullptr;
  std::string engine_identity, model_name = "model";
  int max_model_len = 0;
  pid_t engine_pid = -1;

  std::mutex mu;
  std::deque<Delta> queue;
  int evfd = -1, epfd = -1, lfd = -1;
  bool engine_dead = false;
  std::map<int, Conn> conns;
  std::map<std::string, Pending> pending;
  long next_id = 0;

  // ---- engine side
  void bind_sockets(const std::string& in_addr, const std::string& out_addr) {
    ctx = z.ctx_new();
    router = z.socket(ctx, ZMQ_ROUTER_);
    pull = z.socket(ctx, ZMQ_PULL_);
    int linger = 0, rcv = 200;
    z.setsockopt(router, ZMQ_LINGER_, &linger, sizeof linger);
    z.setsockopt(pull, ZMQ_LINGER_, &linger, sizeof linger);
    z.setsockopt(router, ZMQ_RCVTIMEO_, &rcv, sizeof rcv);
    z.setsockopt(pull, ZMQ_RCVTIMEO_, &rcv, sizeof rcv);
    if (z.bind(router, in_addr.c_str()) != 0 || z.bind(pull, out_addr.c_str()) != 0)
      throw std::runtime_error(std::string("zmq bind failed: ") + z.strerror(z.zerrno()));
  }
  void spawn_engine(std::string cmd, const std::string& in_addr, const std::string& out_addr) {
    auto sub = [&](const std::string& key, const std::string& v) {
      for (size_t at; (at = cmd.find(key)) != std::string::npos;) cmd.replace(at, key.size(), v);
    };
    sub("{input}", in_addr);
    sub("{output}", out_addr);
    engine_pid = fork();
    if (engine_pid < 0) throw std::runtime_error("fork failed");
    if (engine_pid == 0) {
      execl("/bin/sh", "sh", "-c", cmd.c_str(), (char*)nullptr);
      _exit(127);
    }
  }
  bool engine_exited() {
    if (engine_pid <= 0) return false;
    int st = 0;
    return waitpid(engine_pid, &st, WNOHANG) == engine_pid;
  }
  void handshake(int timeout_s) {
    time_t deadline = time(nullptr) + timeout_s;
    bool ready = false;
    while (!ready) {
      if (g_stop) throw std::runtime_error("interrupted");
      if (time(nullptr) > deadline) throw std::runtime_error("engine core handshake timed out");
      if (engine_exited()) throw std::runtime_error("engine core exited during start-up");
      std::vector<std::string> fr;
      if (!z.recv_multipart(router, fr) || fr.size() < 2) continue;
      Val msg = MsgpackReader(fr[1].data(), fr[1].size()).read();
      const Val* st = msg.get("status");
      if (!st) continue;
      engine_identity = fr[0];
      if (st->s == "HELLO") {
        Val ack = Val::map();
        ack.set("ack", Val::boolean(true));
        z.send_multipart(router, {engine_identity, to_msgpack(ack)});
      } else if (st->s == "READY") {
        if (const Val* m = msg.get("max_model_len")) max_model_len = (int)m->as_int();
        ready = true;
      }
    }
  }
  void output_loop() {
    while (!g_stop) {
      std::vector<std::string> fr;
      if (!z.recv_multipart(pull, fr)) continue;
      std::vector<Delta> batch;
      if (fr[0] == "ENGINE_CORE_DEAD") {
        std::lock_guard<std::mutex> lk(mu);
        engine_dead = true;
      } else {
        try {
          Val msg = MsgpackReader(fr[0].data(), fr[0].size()).read();
          if (const Val* outs = msg.get("outputs"))
            for (auto& o : outs->a) {
              Delta d;
              if (const Val* r = o.get("request_id")) d.request_id = r->s;
              if (const Val* t = o.get("new_token_ids")) for (auto& x : t->a) d.tokens.push_back((int)x.as_int());
              if (const Val* f = o.get("finish_reason")) if (!f->is_nil()) d.finish = (int)f->as_int();
              if (const Val* s = o.get("stop_reason")) if (s->t == Val::STR) d.stop_reason = s->s;
              batch.push_back(std::move(d));
            }
        } catch (const std::exception&) {
          continue;  // not an output message (utility reply): nothing for the HTTP side
        }
        std::lock_guard<std::mutex> lk(mu);
        for (auto& d : batch) queue.push_back(std::move(d));
      }
      uint64_t one = 1;
      if (write(evfd, &one, sizeof one) < 0) {}
    }
  }
  void send_add(const std::string& rid, const std::vector<int>& prompt, const Val& sampling, bool ignore_eos) {
    Val req = Val::map();
    req.set("request_id", Val::str(rid));
    Val ids = Val::array();
    for (int t : prompt) ids.push(Val::integer(t));
    req.set("prompt_token_ids", std::move(ids));
    req.set("sampling_params", sampling);
    struct timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    req.set("arrival_time", Val::number(ts.tv_sec + ts.tv_nsec * 1e-9));
    req.set("eos_token_id", (!ignore_eos && tok.eos_id >= 0) ? Val::integer(tok.eos_id) : Val::nil());
    req.set("priority", Val::integer(0));
    req.set("client_index", Val::integer(0));
    z.send_multipart(router, {engine_identity, std::string(1, '\0'), to_msgpack(req)});
  }
  void send_abort(const std::string& rid) {
    Val ids = Val::array();
    ids.push(Val::str(rid));
    z.send_multipart(router, {engine_identity, std::string(1, '\1'), to_msgpack(ids)});
  }

  // ---- HTTP side
  static void set_nonblock(int fd) { fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK); }
  void listen_on(const std::string& host, int port) {
    lfd = socket(AF_INET, SOCK_STREAM, 0);
    int one = 1;
    setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
    sockaddr_in a;
    memset(&a, 0, sizeof a);
    a.sin_family = AF_INET;
    a.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host.c_str(), &a.sin_addr) != 1) throw std::runtime_error("bad --host (IPv4 address expected)");
    if (bind(lfd, (sockaddr*)&a, sizeof a) != 0 || listen(lfd, 256) != 0) throw std::runtime_error(std::string("cannot listen: ") + strerror(errno));
    set_nonblock(lfd);
    epfd = epoll_create1(0);
    evfd = eventfd(0, EFD_NONBLOCK);
    epoll_event ev;
    ev.events = EPOLLIN;
    ev.data.fd = lfd;
    epoll_ctl(epfd, EPOLL_CTL_ADD, lfd, &ev);
    ev.data.fd = evfd;
    epoll_ctl(epfd, EPOLL_CTL_ADD, evfd, &ev);
  }
  void watch(int fd, bool want_write) {
    epoll_event ev;
    ev.events = EPOLLIN | EPOLLRDHUP | (want_write ? EPOLLOUT : 0);
    ev.data.fd = fd;
    epoll_ctl(epfd, EPOLL_CTL_MOD, fd, &ev);
  }
  void drop(int fd) {
    auto it = conns.find(fd);
    if (it == conns.end()) return;
    if (!it->second.active_request.empty()) {
      auto p = pending.find(it->second.active_request);
      if (p != pending.end()) {
        send_abort(p->first);  // the client went away: stop generating for it
        pending.erase(p);
      }
    }
    epoll_ctl(epfd, EPOLL_CTL_DEL, fd, nullptr);
    close(fd);
    conns.erase(it);
  }
  void flush(Conn& c) {
    while (!c.out.empty()) {
      ssize_t n = send(c.fd, c.out.data(), c.out.size(), MSG_NOSIGNAL);
      if (n > 0) c.out.erase(0, (size_t)n);
      else if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) { watch(c.fd, true); return; }
      else { drop(c.fd); return; }
    }
    watch(c.fd, false);
    if (c.close_after && c.active_request.empty()) drop(c.fd);
  }
  void respond(Conn& c, int code, const std::string& body, const char* ctype = "application/json") {
    const char* reason = code == 200 ? "OK" : code == 400 ? "Bad Request" : code == 404 ? "Not Found" : code == 503 ? "Service Unavailable" : "Error";
    c.out += "HTTP/1.1 " + std::to_string(code) + " " + reason + "\r\nContent-Type: " + ctype + "\r\nContent-Length: " + std::to_string(body.size()) +
             "\r\nConnection: " + (c.close_after ? "close" : "keep-alive") + "\r\n\r\n" + body;
    flush(c);
  }
  void error(Conn& c, int code, const std::string& msg) {
    Val e = Val::map(), inner = Val::map();
    inner.set("message", Val::str(msg));
    inner.set("type", Val::str(code == 400 ? "invalid_request_error" : "server_error"));
    inner.set("code", Val::integer(code));
    e.set("error", std::move(inner));
    respond(c, code, to_json(e));
  }
  static void chunk(std::string& out, const std::string& data) {
    char h[32];
    snprintf(h, sizeof h, "%zx\r\n", data.size());
    out += h;
    out += data;
    out += "\r\n";
  }

  void handle_completion(Conn& c, const Val& body) {
    const Val* prompt = body.get("prompt");
    if (!prompt) return error(c, 400, "missing prompt");
    std::vector<int> ids;
    try {
      if (prompt->t == Val::STR) ids = tok.encode(prompt->s, true);
      else if (prompt->t == Val::ARR) {
        for (auto& x : prompt->a) {
          if (x.t != Val::INT) return error(c, 400, "prompt must be a string or a list of token ids");
          ids.push_back((int)x.i);
        }
      } else return error(c, 400, "prompt must be a string or a list of token ids");
    } catch (const std::exception& e) {
      return error(c, 400, e.what());
    }
    if (ids.empty()) return error(c, 400, "empty prompt");
    for (int t : ids) if (t < 0 || (tok.vocab_size() > 0 && t >= tok.vocab_size())) return error(c, 400, "token id outside the vocabulary");
    Val sp = Val::map();
    auto num = [&](const char* k, bool as_int) {
      const Val* v = body.get(k);
      if (v && v->is_num()) sp.set(k, as_int ? Val::integer(v->as_int()) : Val::number(v->as_double()));
    };
    int max_tokens = 16;
    if (const Val* m = body.get("max_tokens")) if (m->is_num()) max_tokens = (int)m->as_int();
    if (max_tokens < 1) return error(c, 400, "max_tokens must be at least 1");
    if (max_model_len > 0 && (int)ids.size() + 1 > max_model_len) return error(c, 400, "the prompt is longer than the model's context");
    sp.set("max_tokens", Val::integer(max_tokens));
    num("temperature", false); num("top_p", false); num("min_p", false); num("top_k", true); num("seed", true);
    num("presence_penalty", false); num("frequency_penalty", false); num("repetition_penalty", false); num("min_tokens", true);
    bool ignore_eos = false;
    if (const Val* ie = body.get("ignore_eos")) ignore_eos = ie->t == Val::BOOL && ie->b;
    sp.set("ignore_eos", Val::boolean(ignore_eos));
    if (const Val* st = body.get("stop_token_ids")) if (st->t == Val::ARR) sp.set("stop_token_ids", *st);
    sp.set("output_kind", Val::integer(1));
    sp.set("detokenize", Val::boolean(false));
    std::string rid = "cmpl-native-" + std::to_string(next_id++);
    Pending p;
    p.fd = c.fd;
    if (const Val* s = body.get("stream")) p.stream = s->t == Val::BOOL && s->b;
    if (const Val* r = body.get("return_token_ids")) p.echo_ids = r->t == Val::BOOL && r->b;
    p.n_prompt = (int)ids.size();
    p.created = (long)time(nullptr);
    c.active_request = rid;
    if (p.stream) {
      c.out += "HTTP/1.1 200 OK\r\nContent-Type: text/event-stream\r\nCache-Control: no-cache\r\nTransfer-Encoding: chunked\r\nConnection: keep-alive\r\n\r\n";
      flush(c);
    }
    pending[rid] = std::move(p);
    send_add(rid, ids, sp, ignore_eos);
  }

  Val choice(const std::string& text, const char* finish, const std::vector<int>* ids) {
    Val ch = Val::map();
    ch.set("index", Val::integer(0));
    ch.set("text", Val::str(text));
    ch.set("logprobs", Val::nil());
    ch.set("finish_reason", finish ? Val::str(finish) : Val::nil());
    if (ids) {
      Val a = Val::array();
      for (int t : *ids) a.push(Val::integer(t));
      ch.set("token_ids", std::move(a));
    }
    return ch;
  }
  Val envelope(const std::string& rid, const Pending& p, Val ch) {
    Val r = Val::map();
    r.set("id", Val::str(rid));
    r.set("object", Val::str("text_completion"));
    r.set("created", Val::integer(p.created));
    r.set("model", Val::str(model_name));
    Val chs = Val::array();
    chs.push(std::move(ch));
    r.set("choices", std::move(chs));
    return r;
  }
  void on_delta(const Delta& d) {
    auto it = pending.find(d.request_id);
    if (it == pending.end()) return;
    Pending& p = it->second;
    auto ci = conns.find(p.fd);
    if (ci == conns.end()) { pending.erase(it); return; }
    Conn& c = ci->second;
    p.ids.insert(p.ids.end(), d.tokens.begin(), d.tokens.end());
    std::string fresh = p.held + tok.decode(d.tokens);
    size_t ok = d.finish >= 0 ? fresh.size() : utf8_complete_prefix(fresh);  // hold back a split code point until its bytes arrive
    std::string delta_text = fresh.substr(0, ok);
    p.held = fresh.substr(ok);
    p.text += delta_text;
    static const char* kReason[] = {"stop", "length", "abort", "error"};
    const char* fin = d.finish >= 0 && d.finish < 4 ? kReason[d.finish] : nullptr;
    if (p.stream) {
      if (!delta_text.empty() || fin || !d.tokens.empty()) {
        Val e = envelope(d.request_id, p, choice(delta_text, fin, p.echo_ids ? &d.tokens : nullptr));
        chunk(c.out, "data: " + to_json(e) + "\n\n");
      }
      if (fin) {
        chunk(c.out, "data: [DONE]\n\n");
        c.out += "0\r\n\r\n";
      }
    } else if (fin) {
      Val e = envelope(d.request_id, p, choice(p.text, fin, p.echo_ids ? &p.ids : nullptr));
      Val u = Val::map();
      u.set("prompt_tokens", Val::integer(p.n_prompt));
      u.set("completion_tokens", Val::integer((int64_t)p.ids.size()));
      u.set("total_tokens", Val::integer(p.n_prompt + (int64_t)p.ids.size()));
      e.set("usage", std::move(u));
      if (d.finish == 3) {
        c.active_request.clear();
        pending.erase(it);
        return error(c, 400, d.stop_reason.empty() ? "the engine rejected the request" : d.stop_reason);
      }
      std::string body = to_json(e);
      c.out += "HTTP/1.1 200 OK\r\nContent-Type: application/json\r\nContent-Length: " + std::to_string(body.size()) +
               "\r\nConnection: " + (c.close_after ? "close" : "keep-alive") + "\r\n\r\n" + body;
    }
    if (fin) {
      c.active_request.clear();
      pending.erase(it);
    }
    flush(c);
  }

  void route(Conn& c, const std::string& method, const std::string& path, const std::string& body) {
    if (method == "GET" && (path == "/health" || path == "/ping")) {
      if (engine_dead) return error(c, 503, "the engine core is dead");
      return respond(c, 200, "{}");
    }
    if (method == "GET" && path == "/v1/models") {
      Val m = Val::map(), data = Val::array(), one = Val::map();
      one.set("id", Val::str(model_name));
      one.set("object", Val::str("model"));
      one.set("owned_by", Val::str("onecat"));
      one.set("max_model_len", Val::integer(max_model_len));
      data.push(std::move(one));
      m.set("object", Val::str("list"));
      m.set("data", std::move(data));
      return respond(c, 200, to_json(m));
    }
    if (method != "POST") return error(c, 404, "no such route");
    Val j;
    try {
      j = JsonParser(body).parse();
    } catch (const std::exception& e) {
      return error(c, 400, e.what());
    }
    if (j.t != Val::MAP) return error(c, 400, "the body must be a JSON object");
    if (path == "/tokenize") {
      const Val* t = j.get("prompt") ? j.get("prompt") : j.get("text");
      if (!t || t->t != Val::STR) return error(c, 400, "missing prompt");
      bool special = true;
      if (const Val* a = j.get("add_special_tokens")) special = !(a->t == Val::BOOL && !a->b);
      try {
        std::vector<int> ids = tok.encode(t->s, special);
        Val r = Val::map(), arr = Val::array();
        for (int x : ids) arr.push(Val::integer(x));
        r.set("tokens", std::move(arr));
        r.set("count", Val::integer((int64_t)ids.size()));
        r.set("max_model_len", Val::integer(max_model_len));
        return respond(c, 200, to_json(r));
      } catch (const std::exception& e) {
        return error(c, 400, e.what());
      }
    }
    if (path == "/detokenize") {
      const Val* t = j.get("tokens");
      if (!t || t->t != Val::ARR) return error(c, 400, "missing tokens");
      std::vector<int> ids;
      for (auto& x : t->a) ids.push_back((int)x.as_int());
      Val r = Val::map();
      r.set("prompt", Val::str(tok.decode(ids)));
      return respond(c, 200, to_json(r));
    }
    if (path == "/v1/completions") {
      if (engine_dead) return error(c, 503, "the engine core is dead");
      return handle_completion(c, j);
    }
    return error(c, 404, "no such route");
  }

  void on_readable(int fd) {
    auto it = conns.find(fd);
    if (it == conns.end()) return;
    Conn& c = it->second;
    char buf[65536];
    while (true) {
      ssize_t n = recv(fd, buf, sizeof buf, 0);
      if (n > 0) { c.in.append(buf, (size_t)n); if (c.in.size() > (64u << 20)) return drop(fd); continue; }
      if (n == 0) return drop(fd);
      if (errno == EAGAIN || errno == EWOULDBLOCK) break;
      return drop(fd);
    }
    parse_requests(fd);
  }
  void parse_requests(int fd) {
    while (true) {
      auto it = conns.find(fd);
      if (it == conns.end()) return;
      Conn& c = it->second;
      if (!c.active_request.empty()) return;  // one request at a time per connection
      size_t he = c.in.find("\r\n\r\n");
      if (he == std::string::npos) return;
      std::string head = c.in.substr(0, he);
      size_t le = head.find("\r\n");
      std::string line = head.substr(0, le);
      size_t s1 = line.find(' '), s2 = line.rfind(' ');
      if (s1 == std::string::npos || s2 == s1) return drop(fd);
      std::string method = line.substr(0, s1), path = line.substr(s1 + 1, s2 - s1 - 1);
      size_t q = path.find('?');
      if (q != std::string::npos) path.erase(q);
      size_t clen = 0;
      std::string lower;
      for (char ch : head) lower += (char)tolower((unsigned char)ch);
      size_t cl = lower.find("\r\ncontent-length:");
      if (cl != std::string::npos) clen = (size_t)strtoull(lower.c_str() + cl + 17, nullptr, 10);
      if (lower.find("\r\nconnection: close") != std::string::npos) c.close_after = true;
      if (c.in.size() < he + 4 + clen) return;
      std::string body = c.in.substr(he + 4, clen);
      c.in.erase(0, he + 4 + clen);
      route(c, method, path, body);
    }
  }

  void run() {
    std::thread outs([this] { output_loop(); });
    epoll_event evs[128];
    while (!g_stop) {
      int n = epoll_wait(epfd, evs, 128, 250);
      if (engine_pid > 0 && engine_exited()) {
        engine_dead = true;
        engine_pid = -1;
        fprintf(stderr, "onecat-frontend: the engine core exited\n");
        g_stop = true;
      }
      for (int k = 0; k < n; ++k) {
        int fd = evs[k].data.fd;
        if (fd == lfd) {
          while (true) {
            int cfd = accept(lfd, nullptr, nullptr);
            if (cfd < 0) break;
            set_nonblock(cfd);
            int one = 1;
            setsockopt(cfd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
            epoll_event ev;
            ev.events = EPOLLIN | EPOLLRDHUP;
            ev.data.fd = cfd;
            epoll_ctl(epfd, EPOLL_CTL_ADD, cfd, &ev);
            conns[cfd].fd = cfd;
          }
        } else if (fd == evfd) {
          uint64_t cnt;
          if (read(evfd, &cnt, sizeof cnt) < 0) {}
          std::deque<Delta> got;
          {
            std::lock_guard<std::mutex> lk(mu);
            got.swap(queue);
          }
          for (auto& d : got) {
            int owner = -1;
            auto p = pending.find(d.request_id);
            if (p != pending.end()) owner = p->second.fd;
            on_delta(d);
            if (d.finish >= 0 && owner >= 0) parse_requests(owner);  // a request that arrived while this one ran
          }
        } else {
          if (evs[k].events & (EPOLLHUP | EPOLLERR)) { drop(fd); continue; }
          if (evs[k].events & EPOLLOUT) { auto it = conns.find(fd); if (it != conns.end()) flush(it->second); }
          if (evs[k].events & (EPOLLIN | EPOLLRDHUP)) on_readable(fd);
        }
      }
    }
    g_stop = true;
    outs.join();
  }

  void shutdown() {
    if (engine_pid > 0) {
      // ask the engine to leave its loop, then make sure the exact child this program started is gone
      Val call = Val::array();
      call.push(Val::integer(0));
      call.push(Val::str("shutdown"));
      call.push(Val::array());
      z.send_multipart(router, {engine_identity, std::string(1, '\3'), to_msgpack(call)});
      for (int k = 0; k < 50 && !engine_exited(); ++k) usleep(100000);
      if (engine_pid > 0 && !engine_exited()) { kill(engine_pid, SIGTERM); waitpid(engine_pid, nullptr, 0); }
    }
    for (auto& kv : conns) close(kv.first);
    if (router) z.close(router);
    if (pull) z.close(pull);
    if (ctx) z.ctx_term(ctx);
  }
};

std::string arg_of(int argc, char** argv, const char* name, const char* dflt) {
  for (int i = 1; i + 1 < argc; ++i)
    if (!strcmp(argv[i], name)) return argv[i + 1];
  return dflt;
}
bool has_flag(int argc, char** argv, const char* name) {
  for (int i = 1; i < argc; ++i)
    if (!strcmp(argv[i], name)) return true;
  return false;
}

}  // namespace

int main(int argc, char** argv) {
  try {
    Server s;
    s.tok.load(arg_of(argc, argv, "--tokenizer", "byte"));
    if (has_flag(argc, argv, "--tokenize-stdin")) {
      // test mode: one JSON string per line in, {"ids": [...], "pieces": [...], "text": decode(ids)} per line out
      std::string line;
      char buf[1 << 16];
      while (fgets(buf, sizeof buf, stdin)) {
        line = buf;
        while (!line.empty() && (line.back() == '\n' || line.back() == '\r')) line.pop_back();
        Val in = JsonParser(line).parse();
        std::vector<int> ids = s.tok.encode(in.s, false);
        Val out = Val::map(), a = Val::array(), pcs = Val::array();
        for (int t : ids) a.push(Val::integer(t));
        if (s.tok.can_encode) for (auto& p : s.tok.split(in.s)) pcs.push(Val::str(p));
        out.set("ids", std::move(a));
        out.set("pieces", std::move(pcs));
        out.set("text", Val::str(s.tok.decode(ids, false)));
        printf("%s\n", to_json(out).c_str());
        fflush(stdout);
      }
      return 0;
    }
    signal(SIGINT, on_signal);
    signal(SIGTERM, on_signal);
    signal(SIGPIPE, SIG_IGN);
    s.model_name = arg_of(argc, argv, "--served-model-name", "model");
    s.z.load(arg_of(argc, argv, "--zmq-lib", "libzmq.so.5"));
    std::string tag = std::to_string((long)getpid());
    std::string in_addr = arg_of(argc, argv, "--input-addr", ("ipc:///tmp/onecat-fe-in-" + tag).c_str());
    std::string out_addr = arg_of(argc, argv, "--output-addr", ("ipc:///tmp/onecat-fe-out-" + tag).c_str());
    s.bind_sockets(in_addr, out_addr);
    std::string cmd = arg_of(argc, argv, "--engine-cmd", "");
    if (!cmd.empty()) s.spawn_engine(cmd, in_addr, out_addr);
    s.handshake(atoi(arg_of(argc, argv, "--handshake-timeout", "600").c_str()));
    s.listen_on(arg_of(argc, argv, "--host", "127.0.0.1"), atoi(arg_of(argc, argv, "--port", "8000").c_str()));
    fprintf(stderr, "onecat-frontend: serving on %s:%s (engine ready, max_model_len %d)\n", arg_of(argc, argv, "--host", "127.0.0.1").c_str(),
            arg_of(argc, argv, "--port", "8000").c_str(), s.max_model_len);
    s.run();
    s.shutdown();
    if (in_addr.rfind("ipc://", 0) == 0) unlink(in_addr.c_str() + 6);
    if (out_addr.rfind("ipc://", 0) == 0) unlink(out_addr.c_str() + 6);
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "onecat-frontend: %s\n", e.what());
    return 1;
  }
}
