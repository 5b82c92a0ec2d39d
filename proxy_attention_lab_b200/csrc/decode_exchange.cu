// Context-sharded long-context decode: the cross-GPU half, fused into one kernel.
//
// Every GPU holds a slice of every sequence's context and has run the split-KV pass over it
// (paged_decode_kernel, partials in its workspace).  The reference has no multi-device code; its two-pass decode
// (src/pal_core/src/paged_attention_decode_primitive.cpp:163-240, paged_reduce_decode.h.metal:27-129) is the
// single-GPU form of the merge done here across GPUs.
//
// ctx_exchange_combine_kernel does, in one launch per GPU:
//   1. merge this GPU's partitions of each row into one un-normalised (acc, m, l) triple (log-sum-exp merge);
//   2. store the triple straight into EVERY rank's exchange buffer with plain stores through peer-mapped
//      pointers (NVLink), own buffer included;
//   3. when the last CTA has published, fence and write this step's number into every rank's flag word;
//   4. wait - bounded, like every wait in this library - until all ranks' flags show this step;
//   5. merge the gathered triples and write the attention output.
// No multimem / multicast and no TMA or bulk copy touches peer memory: stores out, ordinary loads of local memory in.
//
// Exchange buffer of one rank (same layout on all ranks, zeroed once at set-up, then owned by the kernels):
//   [0, 256)     state: epoch (steps completed), two CTA counters
//   [256, 512)   flags[64]: flags[r] = number of the last step whose triples rank r has delivered here
//   [512, ...)   gather[2][world][rows_capacity][D + 2] floats, double-buffered by step parity
// Why two buffers suffice: rank A stores step e into B's buffer e & 1.  B read that buffer last in step e - 2; A can
// only reach step e after its step e - 1 kernel saw B's flag e - 1, which B wrote in its step e - 1 kernel, which the
// stream ordered after B's step e - 2 kernel.
// The step number lives in device memory and is advanced by the kernel itself, so a captured CUDA graph replays.
// After a timeout the counters and flags are undefined: the exchange has to be set up again (zeroed on all ranks).
#include <math.h>

#include "common.cuh"
#include "launch.h"

namespace pal {
namespace {

constexpr int kMaxPeers = 16;
constexpr int kStateBytes = 256;
constexpr int kFlagBytes = 256;
constexpr int kExchangeThreads = 128;

struct ExchangeState {
  unsigned int epoch;
  unsigned int published;  // CTAs that have stored all their rows this step
  unsigned int finished;   // CTAs that have finished this step
};

struct ExchangeParams {
  PartialsView in;
  int num_parts, head_dim;
  long long rows, rows_capacity;
  int world, rank;
  unsigned char* peer[kMaxPeers];
  void* out;
  int out_f32;
  WaitCtx wait;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(kExchangeThreads, 8) ctx_exchange_combine_kernel(const ExchangeParams p) {
  __shared__ float s_w[1024];
  __shared__ float s_red[8];
  const int tid = threadIdx.x;
  const int D = p.head_dim, pitch = p.head_dim + 2;
  unsigned char* mine = p.peer[p.rank];
  ExchangeState* state = reinterpret_cast<ExchangeState*>(mine);
  const unsigned int* my_flags = reinterpret_cast<const unsigned int*>(mine + kStateBytes);
  // Every CTA reads the step number before any CTA can advance it (that happens when all have finished).
  const unsigned int step = *reinterpret_cast<volatile unsigned int*>(&state->epoch) + 1u;
  const long long slot = (long long)(step & 1u) * p.world;

  // ---- 1 + 2: merge my partitions of each row, store the triple into every rank's buffer ----
  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const float* mr = p.in.m + row * p.in.row_stride_ml;
    const float* lr = p.in.l + row * p.in.row_stride_ml;
    float mx = -INFINITY;
    for (int j = tid; j < p.num_parts; j += kExchangeThreads) mx = fmaxf(mx, mr[j * p.in.part_stride_ml]);
#pragma unroll
    for (int sh = 16; sh >= 1; sh >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
    if ((tid & 31) == 0) s_red[tid >> 5] = mx;
    __syncthreads();
    const float M = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    __syncthreads();
    float den = 0.f;
    for (int j = tid; j < p.num_parts; j += kExchangeThreads) {
      const float mj = mr[j * p.in.part_stride_ml];
      const float w = (mj > -INFINITY) ? __expf(mj - M) : 0.f;
      if (j < 1024) s_w[j] = w;
      den += w * lr[j * p.in.part_stride_ml];
    }
#pragma unroll
    for (int sh = 16; sh >= 1; sh >>= 1) den += __shfl_xor_sync(0xffffffffu, den, sh);
    if ((tid & 31) == 0) s_red[4 + (tid >> 5)] = den;
    __syncthreads();
    const float den_all = (s_red[4] + s_red[5]) + (s_red[6] + s_red[7]);
    const float* ar = p.in.acc + row * p.in.row_stride_acc;
    auto weight = [&](int j) {
      if (j < 1024) return s_w[j];
      const float mj = mr[j * p.in.part_stride_ml];
      return (mj > -INFINITY) ? __expf(mj - M) : 0.f;
    };
    for (int d = tid; d < D; d += kExchangeThreads) {
      // eight partitions' values in flight at a time (the loop is latency-bound); summed in partition order, exactly as
      // lse_combine_kernel does, so that the two forms of the merge agree bit for bit
      float num = 0.f;
      int j = 0;
      for (; j + 8 <= p.num_parts; j += 8) {
        float a[8], w[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          w[k] = weight(j + k);
          a[k] = ar[(long long)(j + k) * p.in.part_stride_acc + d];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (w[k] != 0.f) num = fmaf(w[k], a[k], num);
      }
      for (; j < p.num_parts; ++j) {
        const float w = weight(j);
        if (w != 0.f) num = fmaf(w, ar[(long long)j * p.in.part_stride_acc + d], num);
      }
      for (int r = 0; r < p.world; ++r) {
        float* dst = reinterpret_cast<float*>(p.peer[r] + kStateBytes + kFlagBytes) +
                     ((slot + p.rank) * p.rows_capacity + row) * pitch;
        dst[d] = num;
      }
    }
    if (tid == 0) {
      for (int r = 0; r < p.world; ++r) {
        float* dst = reinterpret_cast<float*>(p.peer[r] + kStateBytes + kFlagBytes) +
                     ((slot + p.rank) * p.rows_capacity + row) * pitch;
        dst[D] = M;
        dst[D + 1] = den_all;
      }
    }
    __syncthreads();  // s_w / s_red are reused by the next row
  }

  // ---- 3: the CTA that publishes last tells every rank that this rank's triples of this step have landed ----
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    if (atomicAdd(&state->published, 1u) == gridDim.x - 1) {
      state->published = 0u;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        st_release_sys(reinterpret_cast<unsigned int*>(p.peer[r] + kStateBytes) + p.rank, step);
    }
  }

  // ---- 4: wait for every rank's triples (flags only ever grow; compare modulo 2^32) ----
  int ok = 1;
  if (tid < p.world) {
    const unsigned int* f = my_flags + tid;
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(f) - step) < 0) {
      if (clock64() - t0 > p.wait.limit_cycles) {
        if (p.wait.status) atomicExch(p.wait.status, kStatusTimeout);
        ok = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  ok = __syncthreads_and(ok);
  if (!ok) return;

  // ---- 5: merge the ranks' triples of each row (loads bypass L1: the lines were written by other GPUs) ----
  const float* gather = reinterpret_cast<const float*>(mine + kStateBytes + kFlagBytes) + slot * p.rows_capacity * pitch;
  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    float M = -INFINITY;
    for (int r = 0; r < p.world; ++r) M = fmaxf(M, __ldcg(gather + ((long long)r * p.rows_capacity + row) * pitch + D));
    float den = 0.f;
    float w[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      w[r] = 0.f;
      if (r < p.world) {
        const float* src = gather + ((long long)r * p.rows_capacity + row) * pitch;
        const float mj = __ldcg(src + D);
        w[r] = (mj > -INFINITY) ? __expf(mj - M) : 0.f;
        den += w[r] * __ldcg(src + D + 1);
      }
    }
    for (int d = tid; d < D; d += kExchangeThreads) {
      float a[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)  // all ranks' values requested before the first is used
        a[r] = r < p.world ? __ldcg(gather + ((long long)r * p.rows_capacity + row) * pitch + d) : 0.f;
      float num = 0.f;
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < p.world && w[r] != 0.f) num = fmaf(w[r], a[r], num);
      const float v = den > 0.f ? num / den : 0.f;
      if (p.out_f32)
        static_cast<float*>(p.out)[row * D + d] = v;
      else
        static_cast<T*>(p.out)[row * D + d] = Mma16816<T>::from_float(v);
    }
  }

  // ---- the CTA that finishes last advances the step number ----
  __syncthreads();
  if (tid == 0) {
    if (atomicAdd(&state->finished, 1u) == gridDim.x - 1) {
      state->finished = 0u;
      state->epoch = step;
    }
  }
}

}  // namespace

size_t exchange_bytes(int world_size, long long rows_capacity, int head_dim) {
  return (size_t)kStateBytes + kFlagBytes + (size_t)2 * world_size * rows_capacity * (head_dim + 2) * sizeof(float);
}

int launch_exchange_combine(const ExchangeArgs& a, cudaStream_t stream) {
  if (a.world_size < 1 || a.world_size > kMaxPeers || a.rank < 0 || a.rank >= a.world_size) {
    set_error("decode_ctx_exchange: world_size must be in [1, %d] and rank inside it", kMaxPeers);
    return -1;
  }
  if (a.rows > a.rows_capacity) {
    set_error("decode_ctx_exchange: %lld rows but the exchange buffers were sized for %lld", a.rows, a.rows_capacity);
    return -1;
  }
  ExchangeParams p;
  p.in = a.in;
  p.num_parts = a.num_parts;
  p.head_dim = a.head_dim;
  p.rows = a.rows;
  p.rows_capacity = a.rows_capacity;
  p.world = a.world_size;
  p.rank = a.rank;
  for (int r = 0; r < kMaxPeers; ++r)
    p.peer[r] = r < a.world_size ? static_cast<unsigned char*>(const_cast<void*>(a.peer_bases[r])) : nullptr;
  for (int r = 0; r < a.world_size; ++r) {
    if (!p.peer[r] || (reinterpret_cast<uintptr_t>(p.peer[r]) & 255)) {
      set_error("decode_ctx_exchange: peer buffer %d is null or not 256-byte aligned", r);
      return -1;
    }
  }
  p.out = a.out;
  p.out_f32 = a.out_f32 ? 1 : 0;
  p.wait = WaitCtx{&static_cast<WorkspaceHeader*>(a.workspace)->status, wait_limit_cycles()};
  // All CTAs must be resident at once (they wait for one another's rows through the flags): one CTA per row up to a
  // grid that surely fits, rows beyond that are looped over.
  long long grid = a.rows;
  const long long max_grid = (long long)cached_sm_count() * 4;
  if (grid > max_grid) grid = max_grid;
  if (grid < 1) return 0;
  if (a.dtype == 0)
    ctx_exchange_combine_kernel<__half><<<(unsigned)grid, kExchangeThreads, 0, stream>>>(p);
  else
    ctx_exchange_combine_kernel<__nv_bfloat16><<<(unsigned)grid, kExchangeThreads, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace pal
