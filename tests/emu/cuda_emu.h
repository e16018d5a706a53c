// CPU emulation of the small part of the CUDA execution model that the HBM-bound kernels of
// amct_b200/csrc/ckpt_formats.cu and kv_quant.cu use, so that their SOURCE -- index arithmetic, vector and scalar
// paths, reductions, launch geometry, argument checks -- can be executed by a CPU test against the golden vectors.
// TEST INFRASTRUCTURE ONLY: tests/test_kernel_source_emulation.py compiles those .cu files with g++ and this header
// force-included; nothing in the product builds, loads or links it.
//
// Model: the threads of a block are host threads; blocks run one after another.  __syncthreads() is a barrier over
// the block, __shfl_xor_sync a barrier-bracketed exchange inside a 32-thread warp (every lane of a warp must take
// part, and threads may leave a kernel early only as whole warps and never before a block barrier -- true for the
// kernels above).  __shared__ becomes a static variable (one block is alive at a time).  The arithmetic intrinsics
// map to the IEEE operations they name (compile with -ffp-contract=off); fmaf is the C library's exact one.
#pragma once
#define AMCT_CUDA_EMU 1          // the few helpers that are one PTX instruction on the GPU state its effect in C++ here
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>

#include <atomic>
#include <cmath>
#include <condition_variable>
#include <mutex>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace emu {

// Sense-reversing barrier: a short spin, then yield; the emulated blocks are far more threads than host cores, so
// a waiting thread must give its core away quickly.
class Barrier {
 public:
  void reset(int n) {
    n_ = n;
    count_.store(0);
    phase_.store(0);
  }
  void wait() {
    const unsigned phase = phase_.load(std::memory_order_acquire);
    if (count_.fetch_add(1, std::memory_order_acq_rel) + 1 == n_) {
      count_.store(0, std::memory_order_relaxed);
      phase_.store(phase + 1, std::memory_order_release);
    } else {
      int spins = 0;
      while (phase_.load(std::memory_order_acquire) == phase) {
        if (++spins > 64) std::this_thread::yield();
      }
    }
  }

 private:
  int n_ = 1;
  std::atomic<int> count_{0};
  std::atomic<unsigned> phase_{0};
};

struct BlockState {
  Barrier block, step;
  Barrier warp[32];
  uint32_t slot[1024];
};

struct ThreadState {
  uint3 tid{0, 0, 0}, bid{0, 0, 0};
  dim3 bdim{1, 1, 1}, gdim{1, 1, 1};
  BlockState* block = nullptr;
};

inline ThreadState& tls() {
  static thread_local ThreadState s;
  return s;
}

inline unsigned as_dim(const dim3& d, int axis) { return axis == 0 ? d.x : axis == 1 ? d.y : d.z; }

// Host threads that live as long as the process and serve every launch (creating a few hundred threads per launch is
// what small launches would otherwise spend their time on).  Leaked on purpose: the workers are detached.
class Pool {
 public:
  void run(int n, const std::function<void(int)>& job) {
    std::unique_lock<std::mutex> lock(m_);
    while ((int)workers_ < n) {
      const int id = workers_++;
      std::thread([this, id] { loop(id); }).detach();
    }
    job_ = &job;
    active_ = n;
    remaining_ = n;
    ++generation_;
    start_.notify_all();
    done_.wait(lock, [&] { return remaining_ == 0; });
  }

 private:
  void loop(int id) {
    uint64_t seen = 0;
    std::unique_lock<std::mutex> lock(m_);
    for (;;) {
      start_.wait(lock, [&] { return generation_ != seen; });
      seen = generation_;
      if (id < active_) {
        const std::function<void(int)>* job = job_;
        lock.unlock();
        (*job)(id);
        lock.lock();
        if (--remaining_ == 0) done_.notify_one();
      }
    }
  }
  std::mutex m_;
  std::condition_variable start_, done_;
  const std::function<void(int)>* job_ = nullptr;
  int workers_ = 0, active_ = 0, remaining_ = 0;
  uint64_t generation_ = 0;
};

inline Pool& pool() {
  static Pool* p = new Pool;
  return *p;
}

// runs `body` once per (block, thread); `threads` is one-dimensional like every launch of the emulated files
inline void launch(dim3 grid, int threads, const std::function<void()>& body) {
  static BlockState state;                       // launches are serial
  state.block.reset(threads);
  state.step.reset(threads);
  for (int w = 0; w < 32; ++w) {
    const int in_warp = threads - w * 32;
    state.warp[w].reset(in_warp >= 32 ? 32 : (in_warp > 0 ? in_warp : 1));
  }
  pool().run(threads, [&](int t) {
    ThreadState& s = tls();
    s.block = &state;
    s.tid = uint3{(unsigned)t, 0, 0};
    s.bdim = dim3((unsigned)threads, 1, 1);
    s.gdim = grid;
    for (unsigned by = 0; by < grid.y; ++by) {
      for (unsigned bx = 0; bx < grid.x; ++bx) {
        s.bid = uint3{bx, by, 0};
        body();
        state.step.wait();                       // next block only when every thread has left this one
      }
    }
  });
}

// dynamic shared memory of the block that is running
inline void* dynamic_smem() {
  alignas(128) static unsigned char buffer[256 * 1024];
  return buffer;
}

// value of lane `src` (index inside the warp), all 32 lanes taking part
inline uint32_t shfl_idx_bits(uint32_t bits, int src) {
  ThreadState& s = tls();
  const unsigned t = s.tid.x;
  s.block->slot[t] = bits;
  s.block->warp[t >> 5].wait();
  const uint32_t other = s.block->slot[(t & ~31u) + ((unsigned)src & 31u)];
  s.block->warp[t >> 5].wait();
  return other;
}

inline uint32_t shfl_xor_bits(uint32_t bits, int lane_mask) {
  ThreadState& s = tls();
  const unsigned t = s.tid.x;
  s.block->slot[t] = bits;
  s.block->warp[t >> 5].wait();
  const uint32_t other = s.block->slot[t ^ (unsigned)lane_mask];
  s.block->warp[t >> 5].wait();
  return other;
}

}  // namespace emu

#undef __shared__
#undef __noinline__
#define __noinline__ __attribute__((noinline))
#undef __launch_bounds__
#define threadIdx (emu::tls().tid)
#define blockIdx (emu::tls().bid)
#define blockDim (emu::tls().bdim)
#define gridDim (emu::tls().gdim)
#define __shared__ static
#define __launch_bounds__(...)
#define __syncthreads() (emu::tls().block->block.wait())

#define AMCT_LAUNCH(grid, threads, stream, args, ...) \
  emu::launch(dim3(grid), (int)(threads), [&] { __VA_ARGS__ args; })
#define AMCT_LAUNCH_SMEM(grid, threads, smem_bytes, stream, args, ...) \
  emu::launch(dim3(grid), (int)(threads), [&] { __VA_ARGS__ args; })
#define AMCT_DYNAMIC_SMEM(type, name) type* name = reinterpret_cast<type*>(emu::dynamic_smem())
#define cudaFuncSetAttribute(...) cudaSuccess
#define cudaGetDevice(p) (*(p) = 0, cudaSuccess)
#define cudaStreamSynchronize(stream) cudaSuccess
#define cudaDeviceGetAttribute(p, attr, dev) (*(p) = 148, cudaSuccess)
#define cudaGetSymbolAddress(pp, symbol) (*(pp) = (void*)(symbol), cudaSuccess)   // a __device__ array is a host array here
#define AMCT_CHECK_LAUNCH() \
  do {                      \
  } while (0)

static inline float __shfl_xor_sync(unsigned, float v, int lane_mask) {
  uint32_t b;
  std::memcpy(&b, &v, 4);
  b = emu::shfl_xor_bits(b, lane_mask);
  std::memcpy(&v, &b, 4);
  return v;
}
static inline unsigned __shfl_xor_sync(unsigned, unsigned v, int lane_mask) { return emu::shfl_xor_bits(v, lane_mask); }
static inline int __shfl_xor_sync(unsigned, int v, int lane_mask) { return (int)emu::shfl_xor_bits((uint32_t)v, lane_mask); }
static inline unsigned __shfl_sync(unsigned, unsigned v, int src) { return emu::shfl_idx_bits(v, src); }
static inline int __shfl_sync(unsigned, int v, int src) { return (int)emu::shfl_idx_bits((uint32_t)v, src); }
static inline float __shfl_sync(unsigned, float v, int src) {
  uint32_t b;
  std::memcpy(&b, &v, 4);
  b = emu::shfl_idx_bits(b, src);
  std::memcpy(&v, &b, 4);
  return v;
}
// Which lanes run together at a given point cannot be known in this model, and shuffles here always involve the whole
// warp: a kernel path that asks is not emulated (the tests keep away from it).
static inline unsigned __activemask() {
  std::fprintf(stderr, "cuda_emu: __activemask() is not emulated\n");
  std::abort();
}
static inline unsigned __byte_perm(unsigned a, unsigned b, unsigned selector) {
  const uint64_t both = ((uint64_t)b << 32) | a;
  unsigned out = 0;
  for (int i = 0; i < 4; ++i) {
    const unsigned sel = (selector >> (4 * i)) & 0xF;
    unsigned byte = (unsigned)(both >> (8 * (sel & 7))) & 0xFF;
    if (sel & 8) byte = (byte & 0x80) ? 0xFF : 0x00;          // replicate the sign bit
    out |= byte << (8 * i);
  }
  return out;
}
static inline float __uint_as_float(unsigned i) {
  float f;
  std::memcpy(&f, &i, 4);
  return f;
}
static inline float __fmul_rn(float a, float b) { return a * b; }
static inline float __fadd_rn(float a, float b) { return a + b; }
static inline float __fsub_rn(float a, float b) { return a - b; }
static inline float __fdiv_rn(float a, float b) { return a / b; }
static inline float __frcp_rn(float a) { return 1.0f / a; }
static inline float __fmaf_rn(float a, float b, float c) { return std::fmaf(a, b, c); }
static inline int __float_as_int(float f) {
  int i;
  std::memcpy(&i, &f, 4);
  return i;
}
static inline unsigned __float_as_uint(float f) {
  unsigned i;
  std::memcpy(&i, &f, 4);
  return i;
}
static inline float __int_as_float(int i) {
  float f;
  std::memcpy(&f, &i, 4);
  return f;
}
static inline int __popc(unsigned v) { return __builtin_popcount(v); }
static inline int __dp4a(int a, int b, int c) {
  for (int i = 0; i < 4; ++i) c += (int)(int8_t)(a >> (8 * i)) * (int)(int8_t)(b >> (8 * i));
  return c;
}
// correctly rounded 1 / sqrt(x): through double, whose error is far below half an fp32 ulp except on measure-zero ties
static inline float __frsqrt_rn(float x) { return (float)(1.0 / std::sqrt((double)x)); }
static inline int atomicOr(int* p, int v) { return __atomic_fetch_or(p, v, __ATOMIC_SEQ_CST); }
static inline int atomicMin(int* p, int v) {
  int old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
  while (old > v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) {
  }
  return old;
}
static inline int atomicMax(int* p, int v) {
  int old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
  while (old < v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) {
  }
  return old;
}
template <typename T> static inline T __ldg(const T* p) { return *p; }
template <typename T> static inline T __ldcs(const T* p) { return *p; }
template <typename T> static inline void __stcs(T* p, T v) { *p = v; }
using std::isfinite;
// CUDA's global integer min / max
static inline int min(int a, int b) { return a < b ? a : b; }
static inline int max(int a, int b) { return a > b ? a : b; }
static inline unsigned min(unsigned a, unsigned b) { return a < b ? a : b; }
static inline unsigned max(unsigned a, unsigned b) { return a > b ? a : b; }
static inline long min(long a, long b) { return a < b ? a : b; }
static inline long max(long a, long b) { return a > b ? a : b; }
static inline long long min(long long a, long long b) { return a < b ? a : b; }
static inline long long max(long long a, long long b) { return a > b ? a : b; }
