// Token-sharding exchanges over NVLink peer memory: every rank owns one exchange buffer that all ranks of the
// node map (CUDA IPC), and the kernels below move the layer's small cross-rank sums by plain peer stores and
// loads — no library collective, so a whole sharded layer step can be captured into a CUDA graph.
//
//   peer_exchange_kernel        sum a (B, chunks, P) partial over chunks, push the (B, P) message into every
//                               rank's slot, wait (bounded) for the other ranks' messages, add the slots of a
//                               rank range in rank order and normalise: all-reduce / exclusive prefix / suffix.
//   peer_allreduce_flat_kernel  in-place two-shot all-reduce of the parameter-gradient region: rank r reduces
//                               slice r from all ranks (peer loads) and writes the result to all ranks.
//
// Synchronisation is by epoch flags in the buffer header, written with st.release.sys after a system fence and
// polled with ld.acquire.sys under a time limit (pom_peer_comm::wait_ns, 2 s by default); the epoch counters live in device memory so a replayed graph
// advances them.  A wait that expires records POM_ERR_TIMEOUT in the status word and the kernel carries on (its
// result is then meaningless, which the host sees from the status word); later kernels skip their waits.
// No TMA and no multicast instruction touches peer memory here.
#include <cstring>
#include <mutex>

#include <cuda_bf16.h>

#include "common.cuh"

using namespace pomh;

namespace {

constexpr int kMaxRanks = POM_PEER_MAX_RANKS;
constexpr int kFlatCtas = POM_PEER_FLAT_CTAS;
constexpr int kFlatThreads = 512;
constexpr int kXchgThreads = 1024;
constexpr unsigned long long kDefaultWaitNs = 2000000000ull;  // pom_peer_comm::wait_ns == 0

// Header at the start of every rank's exchange buffer (POM_PEER_HEADER_BYTES reserved).
struct PeerHeader {
  unsigned ctr_small;                          // epochs of peer_exchange_kernel launched by the owner
  unsigned pad0[63];
  unsigned flag_small[2][kMaxRanks];           // [epoch parity][writer rank]
  unsigned pad1[32];
  unsigned ctr_flat[kFlatCtas];                // epochs of peer_allreduce_flat_kernel, per CTA
  unsigned flag_start[kMaxRanks][kFlatCtas];   // [writer rank][cta]
  unsigned flag_done[kMaxRanks][kFlatCtas];
};
static_assert(sizeof(PeerHeader) <= POM_PEER_HEADER_BYTES, "header region too small");

struct PeerDev {
  char* base[kMaxRanks];
  int rank, world;
  unsigned long long slot_floats, slots_off, flat_off;
  unsigned long long stage_off, result_off;  // bf16 images of the gradient region: local copy, reduced result
  unsigned long long wait_ns;  // limit of every wait on another rank
};

__device__ __forceinline__ PeerHeader* header(const PeerDev& c, int r) {
  return reinterpret_cast<PeerHeader*>(c.base[r]);
}
__device__ __forceinline__ float* slot(const PeerDev& c, int owner, unsigned parity, int writer) {
  return reinterpret_cast<float*>(c.base[owner] + c.slots_off) +
         (static_cast<unsigned long long>(parity) * c.world + writer) * c.slot_floats;
}

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_sys_f4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_f4(float4* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ float ld_sys_f(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Poll until *flag has reached `epoch` (wrap-safe) or the limit passes; false on expiry.
__device__ __forceinline__ bool wait_flag(const unsigned* flag, unsigned epoch, bool skip, unsigned long long limit_ns) {
  if (static_cast<int>(ld_acquire_sys(flag) - epoch) >= 0) return true;
  if (skip) return false;
  const unsigned long long t0 = now_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (static_cast<int>(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (now_ns() - t0 > limit_ns) return false;
    __nanosleep(100);
  }
}

struct XchgDev {
  const float* partial;
  float* out;
  const float* denom;
  float scale;
  int B, chunks, P;
  int lo, hi;  // ranks [lo, hi) enter the sum
};

__global__ void __launch_bounds__(kXchgThreads) peer_exchange_kernel(PeerDev c, XchgDev a, int* status) {
  __shared__ unsigned s_epoch;
  __shared__ int s_fail;
  const int tid = threadIdx.x;
  PeerHeader* mine = header(c, c.rank);
  if (tid == 0) {
    s_epoch = mine->ctr_small + 1;
    mine->ctr_small = s_epoch;
    s_fail = 0;
  }
  __syncthreads();
  const unsigned epoch = s_epoch, parity = epoch & 1u;
  const bool poisoned = *reinterpret_cast<volatile int*>(status) != 0;
  const int n = a.B * a.P;

  // local chunk sums, pushed into this rank's slot on every rank (own included)
  for (int e = tid; e < n; e += kXchgThreads) {
    const int b = e / a.P, p = e - b * a.P;
    const float* src = a.partial + static_cast<long long>(b) * a.chunks * a.P + p;
    float s0 = 0.f, s1 = 0.f;
    int k = 0;
    for (; k + 1 < a.chunks; k += 2) {
      s0 += src[static_cast<long long>(k) * a.P];
      s1 += src[static_cast<long long>(k + 1) * a.P];
    }
    if (k < a.chunks) s0 += src[static_cast<long long>(k) * a.P];
    const float s = s0 + s1;
    for (int q = 0; q < c.world; ++q) slot(c, q, parity, c.rank)[e] = s;
  }
  __threadfence_system();
  __syncthreads();
  if (tid < c.world) st_release_sys(&header(c, tid)->flag_small[parity][c.rank], epoch);
  if (tid < c.world && !wait_flag(&mine->flag_small[parity][tid], epoch, poisoned, c.wait_ns)) s_fail = 1;
  __syncthreads();
  if (s_fail && tid == 0 && !poisoned) atomicCAS(status, 0, POM_ERR_TIMEOUT);

  for (int e = tid; e < n; e += kXchgThreads) {
    float t = 0.f;
    for (int q = a.lo; q < a.hi; ++q) t += ld_sys_f(slot(c, c.rank, parity, q) + e);
    t *= a.scale;
    if (a.denom) {
      const float d = a.denom[e / a.P];
      t = d != 0.f ? t / d : 0.f;
    }
    a.out[e] = t;
  }
}

__global__ void __launch_bounds__(kFlatThreads) peer_allreduce_flat_kernel(PeerDev c, unsigned long long n4, int* status) {
  __shared__ unsigned s_epoch;
  __shared__ int s_fail;
  const int tid = threadIdx.x, cta = blockIdx.x;
  PeerHeader* mine = header(c, c.rank);
  if (tid == 0) {
    s_epoch = mine->ctr_flat[cta] + 1;
    mine->ctr_flat[cta] = s_epoch;
    s_fail = 0;
  }
  __syncthreads();
  const unsigned epoch = s_epoch;
  const bool poisoned = *reinterpret_cast<volatile int*>(status) != 0;

  // every rank's gradients are complete once its kernel has started (stream order)
  if (tid < c.world) st_release_sys(&header(c, tid)->flag_start[c.rank][cta], epoch);
  if (tid < c.world && !wait_flag(&mine->flag_start[tid][cta], epoch, poisoned, c.wait_ns)) s_fail = 1;
  __syncthreads();

  const unsigned long long per = (n4 + c.world - 1) / c.world;
  const unsigned long long lo = per * c.rank;
  const unsigned long long hi = lo + per < n4 ? lo + per : n4;
  float4* buf[kMaxRanks];
#pragma unroll
  for (int q = 0; q < kMaxRanks; ++q)
    buf[q] = q < c.world ? reinterpret_cast<float4*>(c.base[q] + c.flat_off) : nullptr;
  if (!s_fail) {
    for (unsigned long long i = lo + static_cast<unsigned long long>(cta) * kFlatThreads + tid; i < hi;
         i += static_cast<unsigned long long>(kFlatCtas) * kFlatThreads) {
      float4 v[kMaxRanks];
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q)
        if (q < c.world) v[q] = ld_sys_f4(buf[q] + i);
      float4 acc = v[0];
#pragma unroll
      for (int q = 1; q < kMaxRanks; ++q)
        if (q < c.world) {
          acc.x += v[q].x;
          acc.y += v[q].y;
          acc.z += v[q].z;
          acc.w += v[q].w;
        }
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q)
        if (q < c.world) st_sys_f4(buf[q] + i, acc);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < c.world) st_release_sys(&header(c, tid)->flag_done[c.rank][cta], epoch);
  if (tid < c.world && !wait_flag(&mine->flag_done[tid][cta], epoch, poisoned || s_fail, c.wait_ns)) s_fail = 1;
  __syncthreads();
  if (s_fail && tid == 0 && !poisoned) atomicCAS(status, 0, POM_ERR_TIMEOUT);
}

// The same all-reduce with bf16 on the wire: the layer's parameters (and so the gradients it hands back) are bf16,
// so each rank first rounds its fp32 accumulators to bf16 into a staging image (local traffic only), rank r then
// pulls slice r of every rank's image, adds in fp32 in rank order, and writes the bf16 sum into every rank's result
// image.  Half the NVLink bytes of the fp32 form, and the separate fp32 -> bf16 cast of the result disappears.
// One work unit = 8 values (32 bytes fp32, 16 bytes bf16).  CTA c converts, in every slice, exactly the units that
// CTA c of the owning rank will pull, so the per-CTA start flags cover the dependency.
__device__ __forceinline__ uint4 ld_sys_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_u4(uint4* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ unsigned pack2_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&h);
}

__global__ void __launch_bounds__(kFlatThreads) peer_allreduce_flat_bf16_kernel(PeerDev c, unsigned long long n8,
                                                                                int* status) {
  __shared__ unsigned s_epoch;
  __shared__ int s_fail;
  const int tid = threadIdx.x, cta = blockIdx.x;
  PeerHeader* mine = header(c, c.rank);
  if (tid == 0) {
    s_epoch = mine->ctr_flat[cta] + 1;
    mine->ctr_flat[cta] = s_epoch;
    s_fail = 0;
  }
  __syncthreads();
  const unsigned epoch = s_epoch;
  const bool poisoned = *reinterpret_cast<volatile int*>(status) != 0;
  const unsigned long long per = (n8 + c.world - 1) / c.world;
  const unsigned long long stride = static_cast<unsigned long long>(kFlatCtas) * kFlatThreads;
  const unsigned long long first = static_cast<unsigned long long>(cta) * kFlatThreads + tid;

  // local image: fp32 accumulators -> bf16, slice by slice with the pull pattern of the reducing rank
  {
    const float4* src = reinterpret_cast<const float4*>(c.base[c.rank] + c.flat_off);
    uint4* dst = reinterpret_cast<uint4*>(c.base[c.rank] + c.stage_off);
    for (int sl = 0; sl < c.world; ++sl) {
      const unsigned long long lo = per * sl, hi = lo + per < n8 ? lo + per : n8;
      for (unsigned long long i = lo + first; i < hi; i += stride) {
        const float4 a = src[2 * i], b = src[2 * i + 1];
        dst[i] = make_uint4(pack2_bf16(a.x, a.y), pack2_bf16(a.z, a.w), pack2_bf16(b.x, b.y), pack2_bf16(b.z, b.w));
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < c.world) st_release_sys(&header(c, tid)->flag_start[c.rank][cta], epoch);
  if (tid < c.world && !wait_flag(&mine->flag_start[tid][cta], epoch, poisoned, c.wait_ns)) s_fail = 1;
  __syncthreads();

  const unsigned long long lo = per * c.rank;
  const unsigned long long hi = lo + per < n8 ? lo + per : n8;
  if (!s_fail) {
    for (unsigned long long i = lo + first; i < hi; i += stride) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      uint4 v[kMaxRanks];
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q)
        if (q < c.world) v[q] = ld_sys_u4(reinterpret_cast<const uint4*>(c.base[q] + c.stage_off) + i);
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q)
        if (q < c.world) {
          const unsigned w[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[2 * e] += __uint_as_float(w[e] << 16);
            acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
          }
        }
      const uint4 out = make_uint4(pack2_bf16(acc[0], acc[1]), pack2_bf16(acc[2], acc[3]), pack2_bf16(acc[4], acc[5]),
                                   pack2_bf16(acc[6], acc[7]));
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q)
        if (q < c.world) st_sys_u4(reinterpret_cast<uint4*>(c.base[q] + c.result_off) + i, out);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < c.world) st_release_sys(&header(c, tid)->flag_done[c.rank][cta], epoch);
  if (tid < c.world && !wait_flag(&mine->flag_done[tid][cta], epoch, poisoned || s_fail, c.wait_ns)) s_fail = 1;
  __syncthreads();
  if (s_fail && tid == 0 && !poisoned) atomicCAS(status, 0, POM_ERR_TIMEOUT);
}

int to_dev(const pom_peer_comm* c, PeerDev* d) {
  if (!c) return POM_ERR_NULL;
  if (c->world < 1 || c->world > kMaxRanks || c->rank < 0 || c->rank >= c->world) return POM_ERR_BAD_SHAPE;
  unsigned long long lay[3];
  int rc = pom_peer_layout(c->world, c->slot_floats, c->flat_floats, lay);
  if (rc) return rc;
  for (int q = 0; q < kMaxRanks; ++q) {
    d->base[q] = q < c->world ? static_cast<char*>(c->base[q]) : nullptr;
    if (q < c->world && (!c->base[q] || !aligned16(c->base[q]))) return POM_ERR_NULL;
  }
  d->rank = c->rank;
  d->world = c->world;
  d->slot_floats = c->slot_floats;
  d->slots_off = lay[0];
  d->flat_off = lay[1];
  d->stage_off = lay[1] + c->flat_floats * sizeof(float);
  d->result_off = d->stage_off + c->flat_floats * 2;
  d->wait_ns = c->wait_ns ? c->wait_ns : kDefaultWaitNs;
  return POM_OK;
}

typedef CUresult (*GetRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

GetRangeFn range_fn() {
  static GetRangeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<GetRangeFn>(p);
  });
  return fn;
}

}  // namespace

extern "C" {

int pom_peer_layout(int world, unsigned long long slot_floats, unsigned long long flat_floats,
                    unsigned long long out[3]) {
  if (!out) return POM_ERR_NULL;
  if (world < 1 || world > kMaxRanks) return POM_ERR_BAD_SHAPE;
  if (slot_floats == 0 || (slot_floats & 3ull) || (flat_floats & 3ull)) return POM_ERR_BAD_ALIGN;
  out[0] = POM_PEER_HEADER_BYTES;
  out[1] = out[0] + 2ull * world * slot_floats * sizeof(float);
  // gradient region: fp32 accumulators, then their bf16 staging image, then the bf16 result image
  out[2] = out[1] + flat_floats * (sizeof(float) + 2 + 2);
  return POM_OK;
}

int pom_peer_export(const void* dev_ptr, void* handle_out, unsigned long long* offset_out) {
  if (!dev_ptr || !handle_out || !offset_out) return POM_ERR_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == POM_PEER_HANDLE_BYTES, "IPC handle size");
  GetRangeFn fn = range_fn();
  if (!fn) return POM_ERR_CUDA;
  CUdeviceptr base = 0;
  size_t size = 0;
  if (fn(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr)) != CUDA_SUCCESS) return POM_ERR_CUDA;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
    cudaGetLastError();
    return POM_ERR_CUDA;
  }
  std::memcpy(handle_out, &h, sizeof(h));
  *offset_out = reinterpret_cast<CUdeviceptr>(dev_ptr) - base;
  return POM_OK;
}

int pom_peer_open(const void* handle, void** base_out) {
  if (!handle || !base_out) return POM_ERR_NULL;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return POM_ERR_CUDA;
  }
  *base_out = p;
  return POM_OK;
}

int pom_peer_close(void* base) {
  if (!base) return POM_ERR_NULL;
  if (cudaIpcCloseMemHandle(base) != cudaSuccess) {
    cudaGetLastError();
    return POM_ERR_CUDA;
  }
  return POM_OK;
}

int pom_peer_exchange(const pom_peer_comm* c, const pom_peer_xchg_args* a, int* status, void* stream) {
  if (!a || !a->partial || !a->out || !status) return POM_ERR_NULL;
  PeerDev d;
  int rc = to_dev(c, &d);
  if (rc) return rc;
  if (a->B <= 0 || a->chunks <= 0 || a->P <= 0) return POM_ERR_BAD_SHAPE;
  if (static_cast<unsigned long long>(a->B) * a->P > c->slot_floats) return POM_ERR_TOO_LARGE;
  XchgDev x;
  x.partial = a->partial;
  x.out = a->out;
  x.denom = a->denom;
  x.scale = a->scale;
  x.B = a->B;
  x.chunks = a->chunks;
  x.P = a->P;
  switch (a->mode) {
    case POM_PEER_SUM_ALL: x.lo = 0; x.hi = c->world; break;
    case POM_PEER_SUM_BEFORE: x.lo = 0; x.hi = c->rank; break;
    case POM_PEER_SUM_AFTER: x.lo = c->rank + 1; x.hi = c->world; break;
    default: return POM_ERR_UNSUPPORTED;
  }
  peer_exchange_kernel<<<1, kXchgThreads, 0, static_cast<cudaStream_t>(stream)>>>(d, x, status);
  count_launch();
  return check_launch();
}

int pom_peer_allreduce_flat(const pom_peer_comm* c, unsigned long long n_floats, int* status, void* stream) {
  if (!status) return POM_ERR_NULL;
  PeerDev d;
  int rc = to_dev(c, &d);
  if (rc) return rc;
  if (n_floats == 0 || (n_floats & 3ull)) return POM_ERR_BAD_ALIGN;
  if (n_floats > c->flat_floats) return POM_ERR_TOO_LARGE;
  peer_allreduce_flat_kernel<<<kFlatCtas, kFlatThreads, 0, static_cast<cudaStream_t>(stream)>>>(d, n_floats / 4,
                                                                                                 status);
  count_launch();
  return check_launch();
}

int pom_peer_allreduce_flat_bf16(const pom_peer_comm* c, unsigned long long n_floats, int* status, void* stream) {
  if (!status) return POM_ERR_NULL;
  PeerDev d;
  int rc = to_dev(c, &d);
  if (rc) return rc;
  if (n_floats == 0 || (n_floats & 7ull) || (c->flat_floats & 7ull)) return POM_ERR_BAD_ALIGN;
  if (n_floats > c->flat_floats) return POM_ERR_TOO_LARGE;
  peer_allreduce_flat_bf16_kernel<<<kFlatCtas, kFlatThreads, 0, static_cast<cudaStream_t>(stream)>>>(d, n_floats / 8,
                                                                                                      status);
  count_launch();
  return check_launch();
}

}  // extern "C"
