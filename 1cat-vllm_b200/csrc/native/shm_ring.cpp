// Native host-side runtime helpers (module onecat_vllm.utils._native):
//   * ShmRing  — single-writer / N-reader broadcast ring in POSIX shared memory, used to fan one RPC out to all worker processes
//     without a socket round trip per worker. Layout: header, then per chunk {seq, len, written flag, one done flag per reader},
//     then the chunk payloads. The writer may reuse a chunk only when every reader has marked it done; readers wait for the
//     written flag of the chunk that matches their own sequence number.
//   * spin_wait — bounded spin on a cache line with pause instructions, falling back to short sleeps, with a deadline.
// Every wait takes a timeout and returns a status instead of blocking forever, so a dead peer surfaces as an error on the host.
// (reference: vllm/distributed/device_communicators/shm_broadcast.py:104,216-260,365 ring buffer and SpinCondition; csrc/spinloop.cpp)
#include <pybind11/pybind11.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#if defined(__x86_64__)
#include <immintrin.h>
static inline void cpu_relax() { _mm_pause(); }
#else
static inline void cpu_relax() { std::this_thread::yield(); }
#endif

namespace py = pybind11;
using Clock = std::chrono::steady_clock;

namespace {

struct Header {
  uint32_t magic;
  uint32_t n_readers;
  uint32_t max_chunks;
  uint32_t chunk_bytes;
  std::atomic<uint64_t> write_seq;  // messages published so far
};

struct ChunkMeta {
  std::atomic<uint64_t> seq;      // sequence number of the message stored here (+1; 0 = never written)
  std::atomic<uint32_t> len;
  std::atomic<uint32_t> done[32];  // done[r] == low 32 bits of seq once reader r consumed it
};

constexpr uint32_t kMagic = 0x0ca7b200;

template <class Pred>
bool wait_until(Pred pred, double timeout_ms) {
  const auto deadline = Clock::now() + std::chrono::microseconds((long long)(timeout_ms * 1000.0));
  for (int spin = 0;; ++spin) {
    if (pred()) return true;
    if (spin < 2000) { cpu_relax(); continue; }
    if (Clock::now() > deadline) return false;
    if (spin < 20000) std::this_thread::yield();
    else std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

class ShmRing {
 public:
  ShmRing(const std::string& name, int n_readers, int max_chunks, int chunk_bytes, bool create)
      : name_(name), owner_(create) {
    if (n_readers < 1 || n_readers > 32) throw std::invalid_argument("n_readers must be in [1, 32]");
    size_t meta = sizeof(Header) + sizeof(ChunkMeta) * (size_t)max_chunks;
    meta = (meta + 63) & ~size_t(63);
    bytes_ = meta + (size_t)max_chunks * (size_t)chunk_bytes;
    int fd = shm_open(name.c_str(), create ? (O_CREAT | O_EXCL | O_RDWR) : O_RDWR, 0600);
    if (fd < 0) throw std::runtime_error("shm_open failed for " + name);
    if (create && ftruncate(fd, (off_t)bytes_) != 0) { close(fd); shm_unlink(name.c_str()); throw std::runtime_error("ftruncate failed"); }
    if (!create) {
      struct stat st;
      if (fstat(fd, &st) != 0 || (size_t)st.st_size < bytes_) { close(fd); throw std::runtime_error("shared segment is smaller than expected"); }
    }
    base_ = (uint8_t*)mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (base_ == MAP_FAILED) throw std::runtime_error("mmap failed");
    hdr_ = reinterpret_cast<Header*>(base_);
    chunks_ = reinterpret_cast<ChunkMeta*>(base_ + sizeof(Header));
    data_ = base_ + meta;
    if (create) {
      std::memset(base_, 0, meta);
      hdr_->n_readers = n_readers; hdr_->max_chunks = max_chunks; hdr_->chunk_bytes = chunk_bytes;
      hdr_->write_seq.store(0);
      std::atomic_thread_fence(std::memory_order_release);
      hdr_->magic = kMagic;
    } else if (hdr_->magic != kMagic || hdr_->n_readers != (uint32_t)n_readers || hdr_->max_chunks != (uint32_t)max_chunks ||
               hdr_->chunk_bytes != (uint32_t)chunk_bytes) {
      munmap(base_, bytes_);
      throw std::runtime_error("shared segment does not match the expected geometry");
    }
  }
  ~ShmRing() {
    if (base_ && base_ != MAP_FAILED) munmap(base_, bytes_);
    if (owner_) shm_unlink(name_.c_str());
  }

  // Publish one message. Returns false if some reader did not free the chunk within the timeout.
  bool write(py::bytes msg, double timeout_ms) {
    char* buf; ssize_t len;
    if (PYBIND11_BYTES_AS_STRING_AND_SIZE(msg.ptr(), &buf, &len) != 0) throw std::runtime_error("bad bytes object");
    if ((size_t)len > hdr_->chunk_bytes) throw std::length_error("message larger than a ring chunk");
    const uint64_t seq = hdr_->write_seq.load(std::memory_order_relaxed);
    ChunkMeta& c = chunks_[seq % hdr_->max_chunks];
    const uint64_t prev = c.seq.load(std::memory_order_acquire);
    bool ok;
    {
      py::gil_scoped_release rel;
      ok = wait_until([&] {
        if (prev == 0) return true;
        for (uint32_t r = 0; r < hdr_->n_readers; ++r)
          if (c.done[r].load(std::memory_order_acquire) != (uint32_t)prev) return false;
        return true;
      }, timeout_ms);
      if (ok) {
        std::memcpy(data_ + (seq % hdr_->max_chunks) * (size_t)hdr_->chunk_bytes, buf, (size_t)len);
        c.len.store((uint32_t)len, std::memory_order_relaxed);
        c.seq.store(seq + 1, std::memory_order_release);
        hdr_->write_seq.store(seq + 1, std::memory_order_release);
      }
    }
    return ok;
  }

  // Next message for reader `r`, or None on timeout.
  py::object read(int r, double timeout_ms) {
    if (r < 0 || (uint32_t)r >= hdr_->n_readers) throw std::out_of_range("reader index");
    const uint64_t want = read_seq_[r] + 1;
    ChunkMeta& c = chunks_[read_seq_[r] % hdr_->max_chunks];
    bool ok;
    {
      py::gil_scoped_release rel;
      ok = wait_until([&] { return c.seq.load(std::memory_order_acquire) == want; }, timeout_ms);
    }
    if (!ok) return py::none();
    const uint32_t len = c.len.load(std::memory_order_relaxed);
    py::bytes out((const char*)(data_ + (read_seq_[r] % hdr_->max_chunks) * (size_t)hdr_->chunk_bytes), len);
    c.done[r].store((uint32_t)want, std::memory_order_release);
    ++read_seq_[r];
    return out;
  }

  uint64_t published() const { return hdr_->write_seq.load(std::memory_order_acquire); }
  int chunk_bytes() const { return (int)hdr_->chunk_bytes; }

 private:
  std::string name_;
  bool owner_;
  size_t bytes_ = 0;
  uint8_t* base_ = nullptr;
  Header* hdr_ = nullptr;
  ChunkMeta* chunks_ = nullptr;
  uint8_t* data_ = nullptr;
  uint64_t read_seq_[32] = {0};
};

// Spin until the 8-byte word at `addr` (inside a Python buffer) differs from `old`, or the timeout passes.
bool spin_wait_changed(py::buffer b, size_t offset, uint64_t old, double timeout_ms) {
  py::buffer_info info = b.request();
  if (offset + 8 > (size_t)info.size * (size_t)info.itemsize) throw std::out_of_range("offset");
  auto* p = reinterpret_cast<std::atomic<uint64_t>*>((uint8_t*)info.ptr + offset);
  py::gil_scoped_release rel;
  return wait_until([&] { return p->load(std::memory_order_acquire) != old; }, timeout_ms);
}

}  // namespace

void register_drafting(py::module_& m);  // ngram.cpp
void register_cpu_attention(py::module_& m);  // cpu_attention.cpp

PYBIND11_MODULE(_native, m) {
  register_drafting(m);
  register_cpu_attention(m);
  py::class_<ShmRing>(m, "ShmRing")
      .def(py::init<const std::string&, int, int, int, bool>(), py::arg("name"), py::arg("n_readers"), py::arg("max_chunks"), py::arg("chunk_bytes"),
           py::arg("create"))
      .def("write", &ShmRing::write, py::arg("msg"), py::arg("timeout_ms") = 10000.0)
      .def("read", &ShmRing::read, py::arg("reader"), py::arg("timeout_ms") = 10000.0)
      .def("published", &ShmRing::published)
      .def_property_readonly("chunk_bytes", &ShmRing::chunk_bytes);
  m.def("spin_wait_changed", &spin_wait_changed, py::arg("buffer"), py::arg("offset"), py::arg("old"), py::arg("timeout_ms") = 1000.0);
}
