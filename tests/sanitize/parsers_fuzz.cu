// Host-only hostile-metadata run of every metadata parser of libhodu_b200, meant to be built
// with -fsanitize=address,undefined (tests/test_sanitize_parsers.py does that): short arrays,
// huge ranks, extents whose products overflow, strides near 2^63.  Each metadata array lives in
// an exactly-sized heap block, so a parser that reads one word too many trips the address
// sanitizer; arithmetic that overflows a signed type trips the undefined-behaviour sanitizer.
// No CUDA device is needed or used: hostile metadata is refused before the device is touched,
// and metadata that is acceptable fails at device selection on a machine without a GPU (on a
// machine with one, this program never launches: all pointers are null or tiny, M*N*K is
// either refused or the call stops at the null-pointer check).
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "../../hodu_b200/csrc/common.cuh"

using namespace hodu_b200;

namespace {
uint64_t g_state = 0x9E3779B97F4A7C15ull;
uint64_t rnd() {  // splitmix64
  uint64_t z = (g_state += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
size_t hostile_word() {
  static const size_t k[] = {0, 1, 2, 3, 4, 7, 8, 16, 17, 18, 19, 31, 64, 128, 255, 4096, 65535, 65536,
                             (size_t)1 << 31, ((size_t)1 << 31) - 1, (size_t)1 << 32, ((size_t)1 << 32) + 1,
                             (size_t)1 << 40, (size_t)1 << 62, (size_t)1 << 63, ((size_t)1 << 63) - 1,
                             ~(size_t)0, ~(size_t)0 - 1, ~(size_t)0 >> 1};
  const uint64_t r = rnd();
  if ((r & 3) == 0) return (size_t)(rnd() % 9);
  if ((r & 3) == 1) return (size_t)rnd();
  return k[(r >> 8) % (sizeof(k) / sizeof(k[0]))];
}
// Exactly `len` words on the heap (len 0 -> a one-byte block whose words must never be read).
struct Heap {
  size_t* p;
  explicit Heap(const std::vector<size_t>& v) {
    p = static_cast<size_t*>(malloc(v.empty() ? 1 : v.size() * sizeof(size_t)));
    if (!v.empty()) memcpy(p, v.data(), v.size() * sizeof(size_t));
  }
  ~Heap() { free(p); }
};

std::vector<size_t> valid_matmul(size_t ln, size_t rn, size_t bn) {
  std::vector<size_t> md = {0, ln, rn, bn};
  std::vector<size_t> ls(ln, 2), rs(rn, 2), bs(bn, 2);
  const size_t M = 1 + rnd() % 5, K = 1 + rnd() % 5, N = 1 + rnd() % 5;
  ls[ln - 2] = M; ls[ln - 1] = K; rs[rn - 2] = K; rs[rn - 1] = N;
  size_t num = M * N;
  for (size_t d = 0; d < bn; ++d) num *= bs[d];
  md[0] = num;
  md.insert(md.end(), ls.begin(), ls.end());
  md.insert(md.end(), rs.begin(), rs.end());
  md.insert(md.end(), bs.begin(), bs.end());
  for (size_t i = 0; i < ln + rn; ++i) md.push_back(1 + rnd() % 7);
  md.push_back(0); md.push_back(0);
  md.push_back(M); md.push_back(K); md.push_back(N);
  return md;
}
std::vector<size_t> valid_einsum() {  // "ij,jk->ik"
  const size_t I = 1 + rnd() % 4, J = 1 + rnd() % 4, K = 1 + rnd() % 4;
  return {I * K, 2, 3, 1, 2, I, K, 2, I, J, J, 1, 0, 0, 1, 2, J, K, K, 1, 0, 1, 2, 1, I, J, K, 0, 2};
}
void mutate(std::vector<size_t>& md) {
  const int n = 1 + (int)(rnd() % 4);
  for (int i = 0; i < n && !md.empty(); ++i) {
    const uint64_t r = rnd();
    switch (r % 5) {
      case 0: md[(r >> 8) % md.size()] = hostile_word(); break;
      case 1: md.pop_back(); break;
      case 2: md.push_back(hostile_word()); break;
      case 3: md.resize((r >> 8) % (md.size() + 1)); break;
      default: md[(r >> 8) % md.size()] += (r >> 20) % 3 - 1; break;
    }
  }
}
}  // namespace

int main(int argc, char** argv) {
  const long iters = argc > 1 ? atol(argv[1]) : 200000;
  long accepted = 0, refused = 0;
  auto tally = [&](int r) { (r == 0 ? accepted : refused)++; };
  const uint8_t dtypes[] = {HODU_DTYPE_BF16, HODU_DTYPE_F16, HODU_DTYPE_F32, HODU_DTYPE_F8E4M3, HODU_DTYPE_I8, HODU_DTYPE_I32, 200};
  for (long it = 0; it < iters; ++it) {
    const uint8_t dt = dtypes[rnd() % 7];
    const bool keep_valid = (rnd() % 8) == 0;
    {  // matmul wire format through the internal parser and through the entry points (null data pointers)
      std::vector<size_t> md = valid_matmul(2 + rnd() % 3, 2 + rnd() % 3, 2 + rnd() % 2);
      if (!keep_valid) mutate(md);
      Heap h(md);
      Problem pb;
      tally(parse_matmul(md.empty() ? nullptr : h.p, md.size(), &pb));
      tally(hodu_b200_matmul(0, nullptr, dt, nullptr, nullptr, nullptr, h.p, md.size()));
      tally(hodu_b200_matmul_ex(0, nullptr, dt, HODU_DTYPE_F32, nullptr, nullptr, nullptr, h.p, md.size(), 1.f, 1.f, 0));
      std::vector<size_t> lin = md;
      lin.push_back(hostile_word()); lin.push_back(hostile_word());
      Heap hl(lin);
      tally(hodu_b200_linear(0, nullptr, dt, nullptr, nullptr, nullptr, nullptr, hl.p, lin.size(), 0));
      tally(hodu_b200_matmul_host(0, dt, dt, nullptr, nullptr, nullptr, h.p, md.size(), 1.f, 1.f));
    }
    {  // dot wire format (also the static entry point and the SwiGLU form)
      std::vector<size_t> md = {1 + rnd() % 9, 1 + rnd() % 9, 1 + rnd() % 9, 9, 1, 9, 1, 0, 0};
      if (!keep_valid) mutate(md);
      Heap h(md);
      Problem pb;
      const int parsed = parse_dot(md.empty() ? nullptr : h.p, md.size(), &pb);
      tally(parsed);
      if (parsed == 0) {  // what the entry points do next with an accepted problem, as far as host code goes
        pb.in_dtype = HODU_DTYPE_F32; pb.out_dtype = HODU_DTYPE_F32;
        (void)gemm_f32_scratch_bytes(pb);
        (void)tc_operand_describable(pb, pb.a, true, 4);
      }
      tally(hodu_b200_dot(0, nullptr, dt, nullptr, nullptr, nullptr, h.p, md.size()));
      tally(hodu_b200_dot_f32_static(0, nullptr, nullptr, nullptr, nullptr, h.p, md.size()));
      tally(hodu_b200_dot_host(0, dt, dt, nullptr, nullptr, nullptr, h.p, md.size(), 1.f, 1.f));
      std::vector<size_t> sw = md;
      while (sw.size() < 12 && (rnd() % 4)) sw.push_back(hostile_word());
      Heap hs(sw);
      tally(hodu_b200_swiglu(0, nullptr, dt, nullptr, nullptr, nullptr, nullptr, hs.p, sw.size(), (uint32_t)(rnd() % 3)));
      std::vector<size_t> mlp = md;
      while (mlp.size() < 13 && (rnd() % 5)) mlp.push_back(hostile_word());
      Heap hm(mlp);
      tally(hodu_b200_swiglu_mlp_host(0, dt, nullptr, nullptr, nullptr, nullptr, nullptr, hm.p, mlp.size(), (uint32_t)(rnd() % 3)));
    }
    {  // cast / contiguous
      const size_t nd = rnd() % 5;
      std::vector<size_t> md = {1, nd};
      size_t prod = 1;
      for (size_t d = 0; d < nd; ++d) { md.push_back(1 + rnd() % 4); prod *= md.back(); }
      for (size_t d = 0; d < nd; ++d) md.push_back(rnd() % 9);
      md.push_back(0);
      md[0] = prod;
      if (!keep_valid) mutate(md);
      Heap h(md);
      tally(hodu_b200_cast(0, nullptr, HODU_DTYPE_F32, dt, nullptr, nullptr, h.p, md.size()));
      tally(hodu_b200_contiguous(0, nullptr, dt, nullptr, nullptr, h.p, md.size()));
    }
    {  // einsum
      std::vector<size_t> md = valid_einsum();
      if (!keep_valid) mutate(md);
      Heap h(md);
      Problem pb;
      bool swapped = false;
      tally(parse_einsum(md.empty() ? nullptr : h.p, md.size(), 2, &pb, &swapped));
      const void* ins[2] = {nullptr, nullptr};
      tally(hodu_b200_einsum(0, nullptr, dt, ins, (size_t)(rnd() % 4), nullptr, h.p, md.size()));
    }
    {  // conv2d
      std::vector<size_t> md = {0, 1 + rnd() % 3, 1 + rnd() % 3, 1 + rnd() % 3, 5, 6, 3, 3, 3, 4, 1, 1, 0, 0, 1, 1, 0, 0};
      md[0] = md[1] * md[3] * md[8] * md[9];
      if (!keep_valid) mutate(md);
      Heap h(md);
      tally(hodu_b200_conv2d(0, nullptr, dt, nullptr, nullptr, nullptr, h.p, md.size()));
    }
  }
  printf("parsers_fuzz: %ld iterations, %ld calls accepted (empty problems), %ld refused, no sanitizer finding\n",
         iters, accepted, refused);
  return 0;
}
