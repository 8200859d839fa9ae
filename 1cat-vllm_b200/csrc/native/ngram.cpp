// Host-side drafting helpers for speculative decoding (no GPU work):
//  * ngram_propose: prompt lookup inside one request's own context: the longest suffix (max_n .. min_n tokens) that occurred
//    earlier, most recent occurrence first; returns the up to k tokens that followed it.
//  * SuffixIndex: a bounded log of finished sequences with a hash index over their n-grams, so that a request can draft from what
//    earlier requests produced (a suffix cache shared by all requests of the engine).
// (reference: v1/spec_decode/ngram_proposer.py — numba kernels; v1/spec_decode/suffix_decoding.py)
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <cstring>
#include <unordered_map>
#include <vector>

namespace py = pybind11;

namespace {

std::vector<int32_t> ngram_propose(py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens, int min_n, int max_n, int k) {
  const int32_t* t = tokens.data();
  const long n_tok = (long)tokens.size();
  std::vector<int32_t> out;
  if (k <= 0 || min_n < 1) return out;
  for (long n = std::min<long>(max_n, n_tok - 1); n >= min_n; --n) {
    const int32_t* pat = t + (n_tok - n);
    for (long start = n_tok - n - 1; start >= 0; --start) {
      if (t[start] != pat[0] || std::memcmp(t + start, pat, (size_t)n * sizeof(int32_t)) != 0) continue;
      const long f0 = start + n, f1 = std::min<long>(f0 + k, n_tok);
      out.assign(t + f0, t + f1);
      return out;
    }
  }
  return out;
}

class SuffixIndex {
 public:
  SuffixIndex(int min_n, int max_n, long max_tokens) : min_n_(min_n), max_n_(max_n), cap_(max_tokens) {}

  // Appends one finished sequence and indexes every position by the n-grams that end just before it.
  void add(py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens) {
    const long n = (long)tokens.size();
    if (n <= min_n_) return;
    if ((long)log_.size() + n + 1 > cap_) {  // bounded memory: start over rather than evict piecemeal
      log_.clear();
      index_.clear();
    }
    if (n + 1 > cap_) return;
    const long base = (long)log_.size();
    log_.insert(log_.end(), tokens.data(), tokens.data() + n);
    log_.push_back(kSep);
    for (long pos = base + min_n_; pos < base + n; ++pos)          // pos: first token of the continuation
      for (int g = min_n_; g <= max_n_ && pos - g >= base; ++g) index_[key(&log_[pos - g], g)] = pos;
    ++sequences_;
  }

  // Longest suffix of `context` (max_n .. min_n) found in the log: returns up to k tokens that followed its latest occurrence.
  std::vector<int32_t> propose(py::array_t<int32_t, py::array::c_style | py::array::forcecast> context, int k) const {
    std::vector<int32_t> out;
    const int32_t* c = context.data();
    const long n = (long)context.size();
    for (int g = (int)std::min<long>(max_n_, n); g >= min_n_; --g) {
      auto it = index_.find(key(c + n - g, g));
      if (it == index_.end()) continue;
      const long pos = it->second;
      if (std::memcmp(&log_[pos - g], c + n - g, (size_t)g * sizeof(int32_t)) != 0) continue;  // hash collision
      for (long p = pos; p < (long)log_.size() && (long)out.size() < k && log_[p] != kSep; ++p) out.push_back(log_[p]);
      if (!out.empty()) return out;
    }
    return out;
  }

  long num_tokens() const { return (long)log_.size(); }
  long num_sequences() const { return sequences_; }

 private:
  static constexpr int32_t kSep = INT32_MIN;
  static uint64_t key(const int32_t* p, int g) {
    uint64_t h = 0xcbf29ce484222325ull ^ (uint64_t)g;
    for (int i = 0; i < g; ++i) {
      h ^= (uint32_t)p[i];
      h *= 0x100000001b3ull;
    }
    return h;
  }
  int min_n_, max_n_;
  long cap_, sequences_ = 0;
  std::vector<int32_t> log_;
  std::unordered_map<uint64_t, long> index_;
};

}  // namespace

void register_drafting(py::module_& m) {
  m.def("ngram_propose", &ngram_propose, py::arg("tokens"), py::arg("min_n"), py::arg("max_n"), py::arg("k"));
  py::class_<SuffixIndex>(m, "SuffixIndex")
      .def(py::init<int, int, long>(), py::arg("min_n"), py::arg("max_n"), py::arg("max_tokens"))
      .def("add", &SuffixIndex::add)
      .def("propose", &SuffixIndex::propose, py::arg("context"), py::arg("k"))
      .def_property_readonly("num_tokens", &SuffixIndex::num_tokens)
      .def_property_readonly("num_sequences", &SuffixIndex::num_sequences);
}
