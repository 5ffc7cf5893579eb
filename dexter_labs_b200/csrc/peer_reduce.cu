// Sum of the row-parallel partial outputs over the ranks of one NVLink domain, for the
// small messages of the few-token regime (83 x 3072 bf16 = 0.5 MB), where a library
// all-reduce is mostly latency.
//
// One-shot push over peer memory.  Every rank owns a region of peer-mapped ("symmetric")
// memory with the same layout:
//     [ control: epoch, exit count ][ flags: world x kBlocks ][ recv: 2 x world x capacity bf16 ]
// Block b of rank r copies its slice of r's partial output into slot r of EVERY rank's
// receive buffer (plain 16-byte stores over NVLink; parity = epoch & 1), fences at system
// scope and writes the epoch into flag [r][b] of every rank.  It then waits (bounded) until
// its own flags [0..world)[b] have reached the epoch, i.e. block b of every rank has delivered the
// same slice, adds the world slots in rank order in fp32 (every rank computes the same
// bits) and writes bf16.  No block waits for another block of its own grid, so the grid
// needs no co-residency; ranks wait for each other only through the flags, and each rank
// runs on its own GPU.
//
// Buffer reuse: the receive buffer alternates with the epoch.  A rank can only start call
// k+1 after its call k, for which it waited for every peer's call-k flags; a peer sends
// those only after finishing call k-1.  So when a rank overwrites parity (k+1)&1 = (k-1)&1,
// every peer has finished reading call k-1.  The epoch lives in the region and is advanced
// by the last block to finish, so replaying a captured CUDA graph (same arguments every
// time) keeps working.
//
// Only plain peer loads/stores and system-scope fences: no multimem, no TMA.
#include <cstdint>
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/dexter_b200.h"

namespace dx {
unsigned wait_tries();  // wq_gemm.cu: polls before a wait on a peer gives up

constexpr int kPeerBlocks = 128;     // grid of every rank (must be equal on all ranks)
constexpr int kPeerThreads = 128;    // 128 threads x <= 32 registers: a block fits beside a GEMM CTA on the same SM
constexpr int kPeerMaxWorld = 8;
constexpr size_t kPeerControlBytes = 256;
constexpr size_t kPeerFlagBytes = static_cast<size_t>(kPeerMaxWorld) * kPeerBlocks * sizeof(unsigned);

struct PeerParams {
  unsigned char* region[kPeerMaxWorld];  // every rank's region as mapped in this process
  const uint4* partial;                  // local [elems] bf16
  uint4* out;                            // local [elems] bf16
  int* status;                           // local error word (may be null)
  long long vecs;                        // elems / 8
  long long capacity_vecs;               // capacity / 8
  int rank, world;
  unsigned wait_tries;                   // polls of ~0.25 us before the wait for a peer gives up
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __uint_as_float(w[i] << 16);
    acc[2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

__global__ void __launch_bounds__(kPeerThreads, 16)
peer_allreduce_kernel(const __grid_constant__ PeerParams P) {
  __shared__ int ok_s;
  unsigned char* mine = P.region[P.rank];
  unsigned* control = reinterpret_cast<unsigned*>(mine);
  const unsigned epoch = control[0] + 1;  // advanced only after every block has read it (below)
  const int b = static_cast<int>(blockIdx.x);
  const size_t recv_off = kPeerControlBytes + kPeerFlagBytes;
  const long long slot_vecs = P.capacity_vecs;
  const long long parity_vecs = slot_vecs * P.world;
  const long long base = static_cast<long long>(epoch & 1u) * parity_vecs;

  // this block's slice
  const long long per = (P.vecs + gridDim.x - 1) / gridDim.x;
  const long long lo = per * b;
  const long long hi = (lo + per) < P.vecs ? (lo + per) : P.vecs;

  // phase 0: deliver the slice to slot `rank` of every rank (own region included)
  for (long long i = lo + threadIdx.x; i < hi; i += kPeerThreads) {
    const uint4 v = P.partial[i];
    for (int r = 0; r < P.world; ++r) {
      uint4* dst = reinterpret_cast<uint4*>(P.region[r] + recv_off) + base + slot_vecs * P.rank;
      dst[i] = v;
    }
  }
  // The barrier orders every thread's stores before the flag writers; their release at system
  // scope is cumulative, so it covers the whole block's stores.
  __syncthreads();
  if (threadIdx.x < P.world) {
    unsigned* flag = reinterpret_cast<unsigned*>(P.region[threadIdx.x] + kPeerControlBytes) +
                     P.rank * kPeerBlocks + b;
    st_release_sys(flag, epoch);
  }
  // phase 1: wait for block b of every rank (bounded: about a second)
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < P.world) {
    const unsigned* flag = reinterpret_cast<const unsigned*>(mine + kPeerControlBytes) +
                           threadIdx.x * kPeerBlocks + b;
    bool ok = false;
    for (unsigned tries = 0; tries < P.wait_tries; ++tries) {
      // >=: a peer may already have gone on to the next call (it cannot be further ahead)
      if (static_cast<int>(ld_acquire_sys(flag) - epoch) >= 0) { ok = true; break; }
      __nanosleep(tries < 64 ? 32 : 256);
    }
    if (!ok) ok_s = 0;
  }
  __syncthreads();
  if (ok_s) {
    const uint4* recv = reinterpret_cast<const uint4*>(mine + recv_off) + base;
    for (long long i = lo + threadIdx.x; i < hi; i += kPeerThreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < P.world; ++r) add_bf16x8(acc, __ldcg(recv + slot_vecs * r + i));
      uint4 o;
      unsigned* ow = reinterpret_cast<unsigned*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 pr = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        ow[j] = *reinterpret_cast<const unsigned*>(&pr);
      }
      P.out[i] = o;
    }
  } else if (threadIdx.x == 0 && P.status) {
    atomicExch(P.status, DXB_ERR_KERNEL_TIMEOUT);
  }
  // the last block to finish advances the epoch for the next call
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(control + 1, 1u) == gridDim.x - 1) {
      control[1] = 0;
      __threadfence();
      control[0] = epoch;
    }
  }
}

}  // namespace dx

extern "C" {

size_t dxb_peer_allreduce_bytes(int world, int64_t capacity_elems) {
  if (world < 1 || world > dx::kPeerMaxWorld || capacity_elems <= 0) return 0;
  const size_t cap = (static_cast<size_t>(capacity_elems) + 7) / 8 * 8;
  return dx::kPeerControlBytes + dx::kPeerFlagBytes + 2 * static_cast<size_t>(world) * cap * 2;
}

int dxb_peer_allreduce(const void* partial, void* out, int64_t elems, void* const* peer_regions,
                       int64_t capacity_elems, int rank, int world, void* status,
                       void* cuda_stream) {
  using namespace dx;
  if (!partial || !out || !peer_regions) return DXB_ERR_NULL;
  if (world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world) return DXB_ERR_SHAPE;
  if (elems <= 0 || elems % 8 || capacity_elems % 8 || elems > capacity_elems) return DXB_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(partial) % 16 || reinterpret_cast<uintptr_t>(out) % 16)
    return DXB_ERR_UNSUPPORTED;
  PeerParams P{};
  for (int r = 0; r < world; ++r) {
    if (!peer_regions[r] || reinterpret_cast<uintptr_t>(peer_regions[r]) % 16) return DXB_ERR_NULL;
    P.region[r] = static_cast<unsigned char*>(peer_regions[r]);
  }
  P.partial = static_cast<const uint4*>(partial);
  P.out = static_cast<uint4*>(out);
  P.status = static_cast<int*>(status);
  P.vecs = elems / 8;
  P.capacity_vecs = capacity_elems / 8;
  P.rank = rank;
  P.world = world;
  P.wait_tries = wait_tries();
  static const int blocks = [] {
    const char* e = getenv("DEXTER_B200_PEER_BLOCKS");
    const int v = e ? atoi(e) : kPeerBlocks;
    return (v >= 1 && v <= kPeerBlocks) ? v : kPeerBlocks;
  }();
  peer_allreduce_kernel<<<blocks, kPeerThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(P);
  return cudaGetLastError() == cudaSuccess ? DXB_OK : DXB_ERR_CUDA;
}

}  // extern "C"
