// Paged attention for the CPU backend: causal, GQA, variable-length batches where a request's queries are the last rows of its
// context (decode, chunked prefill over a cached prefix and multi-token verification are one call), with the sliding window, tanh
// soft-capping and per-head sinks of the Gemma / GPT-OSS / Mistral families. One work item per (request, query head); a pool of
// threads takes items from an atomic counter. Keys stream page by page through an online softmax in fp32; K/V may be fp32 or bf16.
// (reference: csrc/cpu/attention.cpp paged_attention_v1 / v2; csrc/cpu/cpu_attn.cpp)
#include <pybind11/pybind11.h>

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

inline float load(const void* base, size_t idx, int bf16) {
  if (!bf16) return reinterpret_cast<const float*>(base)[idx];
  uint32_t bits = (uint32_t)reinterpret_cast<const uint16_t*>(base)[idx] << 16;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}
inline void store(void* base, size_t idx, float v, int bf16) {
  if (!bf16) { reinterpret_cast<float*>(base)[idx] = v; return; }
  uint32_t bits;
  std::memcpy(&bits, &v, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) { reinterpret_cast<uint16_t*>(base)[idx] = (uint16_t)((bits >> 16) | 0x40); return; }  // NaN stays NaN
  bits += 0x7fffu + ((bits >> 16) & 1u);   // round to nearest even
  reinterpret_cast<uint16_t*>(base)[idx] = (uint16_t)(bits >> 16);
}

struct Args {
  const void *q, *kv;
  void* out;
  float* lse;
  const int *block_table, *qsl, *seq_lens;
  const float* sinks;
  long long q_st, q_sh, o_st, o_sh, bt_stride;
  int R, Hq, Hkv, D, bs, window, q_bf16, kv_bf16;
  float scale, softcap;
};

void run_item(const Args& a, int r, int h, std::vector<float>& qf, std::vector<float>& acc) {
  const int q0 = a.qsl[r], q1 = a.qsl[r + 1], S = a.seq_lens[r];
  const int nq = q1 - q0, D = a.D, g = a.Hq / a.Hkv, hk = h / g;
  if (nq <= 0 || S <= 0) return;
  const int* bt = a.block_table + (size_t)r * a.bt_stride;
  const size_t page = (size_t)2 * a.Hkv * a.bs * D;   // elements per block
  for (int i = 0; i < nq; ++i) {
    const int qpos = S - nq + i;
    for (int d = 0; d < D; ++d) qf[d] = load(a.q, (size_t)(q0 + i) * a.q_st + (size_t)h * a.q_sh + d, a.q_bf16) * a.scale;
    float m = -std::numeric_limits<float>::infinity(), l = 0.f;
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    const int lo = a.window > 0 ? std::max(0, qpos - a.window + 1) : 0;
    for (int key = lo; key <= qpos; ++key) {
      const size_t base = (size_t)bt[key / a.bs] * page + ((size_t)hk * a.bs + key % a.bs) * D;
      float s = 0.f;
      for (int d = 0; d < D; ++d) s += qf[d] * load(a.kv, base + d, a.kv_bf16);
      if (a.softcap > 0.f) s = std::tanh(s / a.softcap) * a.softcap;
      if (s > m) {
        const float f = std::exp(m - s);
        l *= f;
        for (int d = 0; d < D; ++d) acc[d] *= f;
        m = s;
      }
      const float p = std::exp(s - m);
      l += p;
      const size_t vbase = base + (size_t)a.Hkv * a.bs * D;
      for (int d = 0; d < D; ++d) acc[d] += p * load(a.kv, vbase + d, a.kv_bf16);
    }
    float lse = m + std::log(l);
    if (a.sinks != nullptr) {   // the sink joins the denominator only
      const float sk = a.sinks[h], mx = std::max(lse, sk);
      const float tot = mx + std::log(std::exp(lse - mx) + std::exp(sk - mx));
      const float keep = std::exp(lse - tot);
      for (int d = 0; d < D; ++d) acc[d] *= keep;
      lse = tot;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int d = 0; d < D; ++d) store(a.out, (size_t)(q0 + i) * a.o_st + (size_t)h * a.o_sh + d, acc[d] * inv, a.q_bf16);
    if (a.lse != nullptr) a.lse[(size_t)(q0 + i) * a.Hq + h] = lse;
  }
}

void cpu_paged_attention(uintptr_t q, uintptr_t kv, uintptr_t out, uintptr_t lse, uintptr_t block_table, uintptr_t qsl, uintptr_t seq_lens, uintptr_t sinks,
                         long long q_st, long long q_sh, long long o_st, long long o_sh, long long bt_stride, int R, int Hq, int Hkv, int D, int bs,
                         double scale, int window, double softcap, int q_bf16, int kv_bf16, int threads) {
  Args a{(const void*)q, (const void*)kv, (void*)out, (float*)lse, (const int*)block_table, (const int*)qsl, (const int*)seq_lens, (const float*)sinks,
         q_st, q_sh, o_st, o_sh, bt_stride, R, Hq, Hkv, D, bs, window, q_bf16, kv_bf16, (float)scale, (float)softcap};
  py::gil_scoped_release nogil;
  const int items = R * Hq;
  int n = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
  n = std::max(1, std::min(n, items));
  std::atomic<int> next{0};
  auto worker = [&]() {
    std::vector<float> qf(D), acc(D);
    for (int it = next.fetch_add(1); it < items; it = next.fetch_add(1)) run_item(a, it / Hq, it % Hq, qf, acc);
  };
  if (n == 1) { worker(); return; }
  std::vector<std::thread> pool;
  for (int t = 0; t < n; ++t) pool.emplace_back(worker);
  for (auto& t : pool) t.join();
}

}  // namespace

void register_cpu_attention(py::module_& m) {
  m.def("cpu_paged_attention", &cpu_paged_attention);
}
