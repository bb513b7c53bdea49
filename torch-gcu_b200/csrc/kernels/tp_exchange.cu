// Tensor-parallel exchange over peer memory (NVLink / NVSwitch), written as this library's own
// kernels instead of a collective library's: what stands where the reference's row-parallel
// projections call ProcessGroupECCL::allreduce (reference:
// torch_gcu/csrc/distributed/ProcessGroupECCL.cpp:2869-2926) and reduce_scatter (:3326-3432).
//
// Every rank maps the other ranks' buffers into its address space once (the host does that with
// IPC handles) and hands the kernels a table of base pointers, its own included. Three pieces:
//
//  * b200_tp_sync: a counting signal / wait between ranks. Rank r owns word [r] of a flag row on
//    every rank; a signal stores r's running count there (fence.sys, then st.release.sys), a wait
//    spins (ld.acquire.sys) until the word written by each peer has reached this rank's running
//    expectation. Counts live in device memory, so a captured graph replays correctly. Every wait
//    is bounded in time: when the bound runs out the kernel sets the TIMEOUT bit of the device
//    error word and returns, it never spins for ever.
//  * b200_tp_reduce_norm: the reduce-scatter, the residual add, the RMSNorm and the all-gather of
//    one row-parallel projection in ONE kernel. The projection of every rank has written its
//    partial product (all rows) into its own peer-visible buffer. This rank owns a block of rows:
//    for each of them it pulls the row from every rank's partial buffer with plain peer loads,
//    sums in fp32 in rank order (deterministic), adds the residual, rounds once (the new residual
//    stream, kept local), normalises, and pushes the normalised row into the gathered activation
//    buffer of every rank with plain peer stores -- so the next column-parallel projection finds
//    all rows locally. No multicast object and no TMA load is involved: peer loads and stores only.
//  * the blocks are small (no shared memory beyond a few words), so they can share an SM with a
//    resident tensor-core GEMM block of another stream instead of needing SMs of their own.
//
// Peer data is read with volatile (L1-bypassing) loads: the L1 of the reading GPU is not coherent
// with writes of another GPU.
#include "common.cuh"

namespace b200 {

unsigned int* device_error_word();  // index.cu

namespace {

constexpr int kTpChannels = 16;
constexpr int kMaxRanks = B200_TP_MAX_RANKS;

struct TpControl {
  unsigned int flags[kTpChannels][kMaxRanks];  // flags[c][r]: written by rank r (peer-visible)
  unsigned int sent[kTpChannels];              // this rank's running signal count, per channel
  unsigned int seen[kTpChannels][kMaxRanks];   // this rank's running expectation of each peer
};

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// One block of 32 threads; thread t talks to rank t.
__global__ void __launch_bounds__(32)
tp_sync_kernel(PeerPtrs control, int world, int rank, int channel, int do_signal, int do_wait,
               unsigned long long timeout_ns, unsigned int* error_word) {
  TpControl* mine = static_cast<TpControl*>(control.p[rank]);
  const int t = threadIdx.x;
  if (do_signal) {
    unsigned int v = 0;
    if (t == 0) {
      v = mine->sent[channel] + 1u;
      mine->sent[channel] = v;
    }
    v = __shfl_sync(0xffffffffu, v, 0);
    // everything this GPU wrote before this kernel (the stream orders it) becomes visible to a
    // peer that acquires the flag
    __threadfence_system();
    if (t < world && t != rank) st_release_sys(&static_cast<TpControl*>(control.p[t])->flags[channel][rank], v);
  }
  if (do_wait && t < world && t != rank) {
    const unsigned int want = mine->seen[channel][t] + 1u;
    mine->seen[channel][t] = want;
    const unsigned int* flag = &mine->flags[channel][t];
    const unsigned long long t0 = global_ns();
    while (static_cast<int>(ld_acquire_sys(flag) - want) < 0) {
      if (global_ns() - t0 > timeout_ns) {
        atomicOr(error_word, 2u);   // bit 1: a bounded wait ran out
        break;
      }
      __nanosleep(64);
    }
  }
}

struct ReduceNormArgs {
  PeerPtrs partial;     // partial.p[r]: rank r's partial product, (total_rows, N) row-major; unused when n_partial == 0
  PeerPtrs gathered;    // gathered.p[r]: rank r's gathered activation buffer, (total_rows, N)
  const void* residual; // (rows, N) local rows of the residual stream, or null
  void* residual_out;   // (rows, N) local; may alias residual; may be null
  const void* weight;   // (N)
  int64_t row0, rows, N;
  int world, rank, n_partial;
  int normalise;        // 0: the gathered rows are the new residual rows themselves
  int gather_all;       // 0: store to this rank's gathered buffer only
  float eps;
};

template <typename T, int BX, int VPT>
__global__ void __launch_bounds__(BX)
tp_reduce_norm_kernel(ReduceNormArgs a) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float smem[BX / 32];
  const int64_t row = blockIdx.x;                 // local row
  const int64_t grow = a.row0 + row;              // row in the full activation
  const int64_t nvec = a.N / V;
  float h[VPT][V];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int64_t vi = threadIdx.x + static_cast<int64_t>(k) * BX;
#pragma unroll
    for (int e = 0; e < V; ++e) h[k][e] = 0.f;
    if (vi < nvec) {
      const int64_t off = (grow * a.N + vi * V) * static_cast<int64_t>(sizeof(T));
      // all peer loads of this vector are issued before the first use
      uint4 part[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < a.n_partial) part[r] = ld_peer16(static_cast<const char*>(a.partial.p[r]) + off);
      Vec16<T> xv;
      if (a.residual) xv = load_stream16(static_cast<const T*>(a.residual) + row * a.N + vi * V);
      float acc[V];
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] = 0.f;
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {   // rank order: the same sum on every run
        if (r < a.n_partial) {
          const Vec16<T>& pv = *reinterpret_cast<const Vec16<T>*>(&part[r]);
#pragma unroll
          for (int e = 0; e < V; ++e) acc[e] += load_as_math(pv.v[e]);
        }
      }
      Vec16<T> hv;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float s = a.residual ? acc[e] + load_as_math(xv.v[e]) : acc[e];
        hv.v[e] = store_from_math<T>(s);
        h[k][e] = load_as_math(hv.v[e]);   // the norm sees the rounded residual stream
        ss += h[k][e] * h[k][e];
      }
      if (a.residual_out) store16(static_cast<T*>(a.residual_out) + row * a.N + vi * V, hv);
    }
  }
  float rstd = 1.f;
  if (a.normalise) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < BX / 32; ++i) tot += smem[i];
    rstd = 1.0f / sqrtf(tot / static_cast<float>(a.N) + a.eps);
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int64_t vi = threadIdx.x + static_cast<int64_t>(k) * BX;
    if (vi < nvec) {
      Vec16<T> o;
      if (a.normalise) {
        Vec16<T> wv = load16(static_cast<const T*>(a.weight) + vi * V);
#pragma unroll
        for (int e = 0; e < V; ++e) o.v[e] = store_from_math<T>(h[k][e] * rstd * load_as_math(wv.v[e]));
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) o.v[e] = store_from_math<T>(h[k][e]);
      }
      const int64_t off = grow * a.N + vi * V;
      if (a.gather_all) {
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < a.world) store16(static_cast<T*>(a.gathered.p[r]) + off, o);
      } else {
        store16(static_cast<T*>(a.gathered.p[a.rank]) + off, o);
      }
    }
  }
}

bool peers_ok(const b200TpPeers* p) {
  if (!p || p->world < 1 || p->world > kMaxRanks || p->rank < 0 || p->rank >= p->world) return false;
  for (int r = 0; r < p->world; ++r)
    if (!p->base[r] || !aligned16(p->base[r])) return false;
  return true;
}

PeerPtrs to_ptrs(const b200TpPeers* p) {
  PeerPtrs o{};
  if (p)
    for (int r = 0; r < p->world && r < kMaxRanks; ++r) o.p[r] = p->base[r];
  return o;
}

template <typename T>
b200Status launch_reduce_norm(const ReduceNormArgs& a, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  const int64_t nvec = a.N / V;
  const unsigned grid = static_cast<unsigned>(a.rows);
  // plain launches (no programmatic dependent launch): the kernel must not start before the wait
  // that precedes it on the stream has completed
  if (nvec <= 256) tp_reduce_norm_kernel<T, 256, 1><<<grid, 256, 0, s>>>(a);
  else if (nvec <= 512) tp_reduce_norm_kernel<T, 256, 2><<<grid, 256, 0, s>>>(a);   // two blocks fit beside a GEMM block
  else if (nvec <= 1024) tp_reduce_norm_kernel<T, 512, 2><<<grid, 512, 0, s>>>(a);
  else if (nvec <= 2048) tp_reduce_norm_kernel<T, 1024, 2><<<grid, 1024, 0, s>>>(a);
  else return fail(B200_NOT_SUPPORTED, "b200_tp_reduce_norm: rows of up to %d elements", 2048 * V);
  return check_launch("b200_tp_reduce_norm");
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_tp_control_bytes(void) { return (sizeof(TpControl) + 255) / 256 * 256; }

b200Status b200_tp_sync(const b200TpPeers* control, int32_t channel, int32_t do_signal, int32_t do_wait,
                        uint64_t timeout_ns, b200Stream stream) {
  B200_REQUIRE(peers_ok(control), B200_BAD_PARAM, "b200_tp_sync: bad peer table");
  B200_REQUIRE(channel >= 0 && channel < kTpChannels, B200_BAD_PARAM, "b200_tp_sync: channel must be in [0, %d)", kTpChannels);
  B200_REQUIRE(timeout_ns > 0, B200_BAD_PARAM, "b200_tp_sync: every wait is bounded: give a positive timeout");
  unsigned int* ew = device_error_word();
  B200_REQUIRE(ew, B200_LAUNCH_FAILED, "b200_tp_sync: device error word unavailable");
  if (control->world == 1 || (!do_signal && !do_wait)) return B200_OK;
  tp_sync_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(to_ptrs(control), control->world, control->rank, channel,
                                                                  do_signal, do_wait, timeout_ns, ew);
  return check_launch("b200_tp_sync");
}

b200Status b200_tp_reduce_norm(const b200TpPeers* partial, const b200TpPeers* gathered, const b200Tensor* residual,
                               const b200Tensor* residual_out, const b200Tensor* weight, int64_t row0, int64_t total_rows,
                               double eps, int32_t normalise, int32_t gather_all, b200Stream stream) {
  B200_REQUIRE(peers_ok(gathered), B200_BAD_PARAM, "b200_tp_reduce_norm: bad table of gathered buffers");
  B200_REQUIRE(!partial || (peers_ok(partial) && partial->world == gathered->world && partial->rank == gathered->rank),
               B200_BAD_PARAM, "b200_tp_reduce_norm: bad table of partial buffers");
  const b200Tensor* shape = residual ? residual : residual_out;
  B200_REQUIRE(shape && valid(shape) && shape->ndim == 2 && is_contiguous(shape), B200_BAD_PARAM,
               "b200_tp_reduce_norm: residual (or residual_out) must be a contiguous (rows, N) view of the local rows");
  B200_REQUIRE(!residual || !residual_out || (same_shape(residual, residual_out) && residual->dtype == residual_out->dtype &&
                                              is_contiguous(residual_out)),
               B200_BAD_PARAM, "b200_tp_reduce_norm: residual_out must match residual");
  B200_REQUIRE(residual || partial, B200_BAD_PARAM, "b200_tp_reduce_norm: nothing to reduce");
  const int64_t rows = shape->sizes[0], N = shape->sizes[1];
  B200_REQUIRE(shape->dtype == B200_BF16 || shape->dtype == B200_F16, B200_NOT_SUPPORTED,
               "b200_tp_reduce_norm: bf16 / f16 activations");
  B200_REQUIRE(N % 8 == 0, B200_NOT_SUPPORTED, "b200_tp_reduce_norm: N must be a multiple of 8");
  B200_REQUIRE(row0 >= 0 && rows >= 0 && row0 + rows <= total_rows, B200_BAD_PARAM, "b200_tp_reduce_norm: row block out of range");
  B200_REQUIRE(!normalise || (weight && valid(weight) && numel(weight) == N && weight->dtype == shape->dtype &&
                              is_contiguous(weight) && aligned16(weight->data)),
               B200_BAD_PARAM, "b200_tp_reduce_norm: weight must be (N) of the activations' dtype");
  B200_REQUIRE((!residual || aligned16(residual->data)) && (!residual_out || aligned16(residual_out->data)), B200_BAD_PARAM,
               "b200_tp_reduce_norm: 16-byte aligned operands");
  if (rows == 0) return B200_OK;
  ReduceNormArgs a{};
  a.partial = to_ptrs(partial);
  a.gathered = to_ptrs(gathered);
  a.residual = residual ? residual->data : nullptr;
  a.residual_out = residual_out ? residual_out->data : nullptr;
  a.weight = weight ? weight->data : nullptr;
  a.row0 = row0;
  a.rows = rows;
  a.N = N;
  a.world = gathered->world;
  a.rank = gathered->rank;
  a.n_partial = partial ? partial->world : 0;
  a.normalise = normalise;
  a.gather_all = gather_all;
  a.eps = static_cast<float>(eps);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (shape->dtype == B200_BF16) return launch_reduce_norm<bf16_t>(a, s);
  return launch_reduce_norm<f16_t>(a, s);
}

}  // extern "C"
