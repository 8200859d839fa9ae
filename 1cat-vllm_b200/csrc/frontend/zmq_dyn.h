// libzmq loaded at run time (the image carries it inside pyzmq's wheel, without headers): the handful of C entry points the
// front end needs, declared here with the constants of zmq.h 4.x.
#pragma once
#include <dlfcn.h>
#include <stddef.h>

#include <stdexcept>
#include <string>
#include <vector>

namespace fe {

struct zmq_msg_t_ { unsigned char _[64]; };
struct zmq_pollitem_t_ { void* socket; int fd; short events; short revents; };

constexpr int ZMQ_DEALER_ = 5, ZMQ_ROUTER_ = 6, ZMQ_PULL_ = 7, ZMQ_PUSH_ = 8;
constexpr int ZMQ_LINGER_ = 17, ZMQ_RCVTIMEO_ = 27, ZMQ_SNDMORE_ = 2, ZMQ_DONTWAIT_ = 1, ZMQ_POLLIN_ = 1, ZMQ_ROUTER_MANDATORY_ = 33;

struct Zmq {
  void* lib = nullptr;
  void* (*ctx_new)() = nullptr;
  int (*ctx_term)(void*) = nullptr;
  void* (*socket)(void*, int) = nullptr;
  int (*close)(void*) = nullptr;
  int (*bind)(void*, const char*) = nullptr;
  int (*setsockopt)(void*, int, const void*, size_t) = nullptr;
  int (*send)(void*, const void*, size_t, int) = nullptr;
  int (*msg_init)(zmq_msg_t_*) = nullptr;
  int (*msg_recv)(zmq_msg_t_*, void*, int) = nullptr;
  void* (*msg_data)(zmq_msg_t_*) = nullptr;
  size_t (*msg_size)(zmq_msg_t_*) = nullptr;
  int (*msg_more)(zmq_msg_t_*) = nullptr;
  int (*msg_close)(zmq_msg_t_*) = nullptr;
  int (*poll)(zmq_pollitem_t_*, int, long) = nullptr;
  int (*zerrno)() = nullptr;
  const char* (*strerror)(int) = nullptr;

  void load(const std::string& path) {
    lib = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (!lib) throw std::runtime_error(std::string("cannot load libzmq (") + path + "): " + dlerror());
    auto sym = [&](const char* n) {
      void* p = dlsym(lib, n);
      if (!p) throw std::runtime_error(std::string("libzmq lacks ") + n);
      return p;
    };
#define ZSYM(field, name) field = reinterpret_cast<decltype(field)>(sym(name))
    ZSYM(ctx_new, "zmq_ctx_new"); ZSYM(ctx_term, "zmq_ctx_term"); ZSYM(socket, "zmq_socket"); ZSYM(close, "zmq_close");
    ZSYM(bind, "zmq_bind"); ZSYM(setsockopt, "zmq_setsockopt"); ZSYM(send, "zmq_send"); ZSYM(msg_init, "zmq_msg_init");
    ZSYM(msg_recv, "zmq_msg_recv"); ZSYM(msg_data, "zmq_msg_data"); ZSYM(msg_size, "zmq_msg_size"); ZSYM(msg_more, "zmq_msg_more");
    ZSYM(msg_close, "zmq_msg_close"); ZSYM(poll, "zmq_poll"); ZSYM(zerrno, "zmq_errno"); ZSYM(strerror, "zmq_strerror");
#undef ZSYM
  }

  // all frames of one message; false on timeout (RCVTIMEO) or error
  bool recv_multipart(void* sock, std::vector<std::string>& frames, int flags = 0) {
    frames.clear();
    while (true) {
      zmq_msg_t_ m;
      msg_init(&m);
      if (msg_recv(&m, sock, flags) < 0) { msg_close(&m); return false; }
      frames.emplace_back((const char*)msg_data(&m), msg_size(&m));
      int more = msg_more(&m);
      msg_close(&m);
      if (!more) return true;
    }
  }
  bool send_multipart(void* sock, const std::vector<std::string>& frames) {
    for (size_t i = 0; i < frames.size(); ++i)
      if (send(sock, frames[i].data(), frames[i].size(), i + 1 < frames.size() ? ZMQ_SNDMORE_ : 0) < 0) return false;
    return true;
  }
};

}  // namespace fe
