// Weight-only quantised GEMM for sm_100a:  Y[M,N] = X[M,K] @ dequant(Q)[K,N] (+ bias)
//
//   Q       packed weights exactly as the reference quantiser lays them out
//           (python/dexter/quant.py:62-133): int4 = [K/2, N] bytes, low nibble is
//           row i, high nibble is row i + K/2 ("split-half"); int8 = [K, N] bytes.
//   scales  [K/G, N] bf16, zeros [K/G, N] bf16 or absent (symmetric).
//   W[k,n]  = bf16( (q - zero) * scale ), one rounding, bit-identical to the
//           reference's torch dequantize (python/dexter/ops/reference/gemm.py:51-73).
//   Y       = bf16( sum_k X*W in fp32 ), then bf16( Y + bias ) as a second rounding,
//           as the reference does (gemm.py:76-79).
//
// Tensor-core kernel (wq_gemm_tc): the weight tile is the 128-row UMMA "M"
// operand and the tokens are the UMMA "N" (swap-AB), so M = 83 tokens costs a
// 96-wide MMA instead of a 128-row one.  24 warps per CTA, one CTA per SM; per unit
// of 128 logical k x 128 columns (64 packed rows of int4, 128 rows of int8):
//   warps 0, 3   TMA producers: packed bytes of alternate units land in a
//                shared-memory ring (128 B swizzle).
//   warp 2       TMA producer: the matching activation k-slices (both nibble planes
//                in one 3-D box for int4).
//   warps 8-23   four dequant teams of four warps, one unit each in flight:
//                ld.shared of packed words, nibble -> bf16 by bit pattern (OR into
//                0x4300 = 128.0, exact subtract, one multiply; no int->float convert),
//                k-pairs formed with two byte permutes, written straight into TMEM with
//                tcgen05.st.16x128b (the dequantised tile never touches shared memory);
//                scales and zero points come from global memory one unit ahead.
//   warp 1       one lane issues tcgen05.mma (A = weights from TMEM, B = activations
//                from shared memory, fp32 accumulators in TMEM, two accumulators).
//   warps 4-7    epilogue: tcgen05.ld, bias, bf16 stores; or fp32 partial sums.
// How the (tile, unit) space is handed to CTAs is chosen per launch (make_plan,
// launch_tc): whole tiles per CTA; equal contiguous unit ranges (stream-K), where a tile
// shared by several CTAs is finished by whichever CTA arrives last (no CTA ever waits for
// another one), summing the partials in a fixed order; or, for few tiles, one
// thread-block cluster per tile that splits K and adds through distributed shared memory.
// More than 128 tokens: every (token block of 128, column tile) pair is a tile, one launch.
#include "wq_common.cuh"

namespace dx {
#ifdef DXB_TRACE
#define DX_DEBUG(bit) (p.debug & (bit))
#define DX_TRACE(role, i) do { if (p.trace && (i) < 32) p.trace[(static_cast<long long>(blockIdx.x) * 8 + (role)) * 32 + (i)] = clock64() - t_start; } while (0)
#else
#define DX_DEBUG(bit) false
#define DX_TRACE(role, i) do { } while (0)
#endif


// ---------------------------------------------------------------------------
// Sum over tensor-parallel ranks fused into the row-parallel GEMM (dxb_gemm_opts.peer_*).
// Every rank owns a region of peer-mapped memory with the same layout:
//   [ control: epoch, exit count ][ arrived: tiles x 8 u32 ][ base: tiles x 8 u32 ]
//   [ recv: 2 parities x world x capacity bf16 ]
// Whoever finishes rows of a 128-column tile (an epilogue warp group or a cluster's owner
// CTA) rounds its fp32 partial sums to bf16 and stores them into slot `rank` of EVERY rank's
// receive buffer (plain 8-byte stores over NVLink, own region included), fences at system
// scope, and adds the number of rows it delivered to arrived[tile][rank] on every rank
// (red.release.sys).  It then waits (bounded) until arrived[tile][s] - base[tile][s] has
// reached the tile's row count for every sender s -- rows are counted, not chunks, so ranks
// may cut their tiles differently -- adds the world slots in rank order in fp32 (every rank
// computes the same bits), applies bias / activation and writes bf16.  The last CTA to
// leave adds the row count to base[][] and advances the epoch (= receive-buffer parity), so
// a captured graph replays.  A rank can be at most one call ahead of a peer, and it then
// writes the other parity.  Only plain peer loads/stores and system-scope fences.
constexpr int kPeerMaxRanks = 8;
constexpr int kFusedMaxTiles = 512;
constexpr size_t kFusedControlBytes = 256;
constexpr size_t kFusedCounterBytes = static_cast<size_t>(kFusedMaxTiles) * kPeerMaxRanks * sizeof(unsigned);
constexpr size_t kFusedHeaderBytes = kFusedControlBytes + 2 * kFusedCounterBytes;

struct PeerFuse {
  unsigned char* region[kPeerMaxRanks];  // every rank's region as mapped in this process
  long long capacity;                    // bf16 elements per receive slot (>= M * N)
  int rank, world;
  unsigned wait_tries;                   // polls of ~0.25 us before a wait gives up
};

__device__ __forceinline__ unsigned* fused_arrived(unsigned char* region, int tile, int sender) {
  return reinterpret_cast<unsigned*>(region + kFusedControlBytes) + tile * kPeerMaxRanks + sender;
}
__device__ __forceinline__ unsigned* fused_base(unsigned char* region, int tile, int sender) {
  return reinterpret_cast<unsigned*>(region + kFusedControlBytes + kFusedCounterBytes) +
         tile * kPeerMaxRanks + sender;
}
__device__ __forceinline__ __nv_bfloat16* fused_recv(const PeerFuse& pf, int owner, unsigned parity, int sender) {
  return reinterpret_cast<__nv_bfloat16*>(pf.region[owner] + kFusedHeaderBytes) +
         (static_cast<long long>(parity) * pf.world + sender) * pf.capacity;
}
__device__ __forceinline__ void red_release_sys_add(unsigned* ptr, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* ptr) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
// Deliver four consecutive columns of one token row to slot `rank` of every rank.
__device__ __forceinline__ void fused_push4(const PeerFuse& pf, unsigned parity, long long elem,
                                            float f0, float f1, float f2, float f3) {
  const uint2 pk = make_uint2(cvt_bf16x2(f1, f0), cvt_bf16x2(f3, f2));
  for (int r = 0; r < pf.world; ++r)
    *reinterpret_cast<uint2*>(fused_recv(pf, r, parity, pf.rank) + elem) = pk;
}
// Tell every rank that `rows` more rows of `tile` from this rank are in place (one thread
// per destination rank; the caller has fenced and synchronised the storing threads).
__device__ __forceinline__ void fused_signal(const PeerFuse& pf, int tile, int dest, unsigned rows) {
  red_release_sys_add(fused_arrived(pf.region[dest], tile, pf.rank), rows);
}
// One thread per sender: bounded wait until that sender's rows of `tile` have all arrived.
__device__ __forceinline__ bool fused_wait(const PeerFuse& pf, int tile, int sender, unsigned rows,
                                           volatile int* abort_flag) {
  unsigned char* mine = pf.region[pf.rank];
  const unsigned base = __ldcg(fused_base(mine, tile, sender));
  const unsigned* arrived = fused_arrived(mine, tile, sender);
  for (unsigned tries = 0; tries < pf.wait_tries; ++tries) {
    if (static_cast<int>(ld_acquire_sys_u32(arrived) - base - rows) >= 0) return true;
    if (*abort_flag) return false;
    __nanosleep(tries < 64 ? 32 : 256);
  }
  *abort_flag = 1;
  return false;
}
// Sum of the world slots for four consecutive columns of one token row, in rank order.
__device__ __forceinline__ float4 fused_sum4(const PeerFuse& pf, unsigned parity, long long elem) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < pf.world; ++s) {
    const uint2 v = __ldcg(reinterpret_cast<const uint2*>(fused_recv(pf, pf.rank, parity, s) + elem));
    acc.x += bf16lo_f32(v.x); acc.y += bf16hi_f32(v.x);
    acc.z += bf16lo_f32(v.y); acc.w += bf16hi_f32(v.y);
  }
  return acc;
}

struct WqParams {
  const __nv_bfloat16* scales;
  const __nv_bfloat16* zeros;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  long long ldo;
  float* partials;
  int* counters;
  int* status;
  int M, N, K, group;
  int NU;              // tokens padded to a multiple of 16: the UMMA N
  int units_per_tile;  // packed rows / 64
  int tiles;           // ceil(N / 128) x token blocks: tile t is token block t / tiles_n,
                       // weight columns 128 * (t % tiles_n)
  int tiles_n;         // ceil(N / 128)
  int total_units;
  int half_k;          // int4: K/2 (first activation column of the high-nibble plane)
  int stages;          // activation (X) ring depth
  int w_stages;        // packed-weight ring depth, a multiple of 4 so that every
                       // stage is only ever used by one dequant team, in order
  int x_stage_bytes;   // planes * NU * 128
  int max_slots;       // partial slots reserved per tile
  int nacc;            // accumulator buffers in TMEM (2 when NU <= 128)
  int group_shift;     // log2(group / 64) when that is a power of two, else -1
  int cluster;         // CTAs per tile (thread-block cluster along x); 1 = no cluster
  int recv_off;        // cluster mode: byte offset of the receive buffers in shared memory
  int recv_alias;      // cluster mode: the receive buffers lie over the (then idle) rings, so
                       // partial rows are only sent once every CTA of the cluster has finished
                       // its main loop
  int rows_per;        // cluster mode: token rows each CTA of the cluster reduces
  int rows_inv;        // ceil(65536 / rows_per): row / rows_per == (row * rows_inv) >> 16
  int epilogue;        // DXB_EPILOGUE_*: what is applied to the bf16 result before it is stored
  int tile_ranges;     // CTAs take whole tiles (ranges cut in tiles, not in units)
  int range_q, range_r;  // quotient and remainder of the cut: units of a tile by the cluster
                         // size, or tiles by the grid size (see the kernel's range arithmetic)
  PeerFuse peer;       // peer.world > 1: the sum over ranks is part of this launch (see below)
  long long* trace;    // only used when built with -DDXB_TRACE
  int debug;           // -DDXB_TRACE builds only: parts of the pipeline to leave out (timing experiments)
};


// tanh-GELU of a value that has already been rounded to bf16, as the reference applies it
// between the FFN linears (torch gelu(approximate="tanh") on the bf16 output of the up
// projection, python/dexter/models/dreamzero/model.py:279-285): evaluated in fp32, rounded once.
__device__ __forceinline__ float gelu_tanh(float v) {
  const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
  return 0.5f * v * (1.0f + tanhf(inner));
}

// Four fp32 sums of one token row -> four bf16 outputs, in the reference's order of
// roundings: round the matmul to bf16, add the bias in bf16 arithmetic (second rounding),
// then the optional activation on that bf16 value (third rounding).
__device__ __forceinline__ uint2 finish_row4(float f0, float f1, float f2, float f3,
                                             const float (&bias4)[4], bool has_bias, int epilogue) {
  uint32_t r01 = cvt_bf16x2(f1, f0), r23 = cvt_bf16x2(f3, f2);
  if (has_bias) {
    const uint32_t b01 = cvt_bf16x2(bf16hi_f32(r01) + bias4[1], bf16lo_f32(r01) + bias4[0]);
    const uint32_t b23 = cvt_bf16x2(bf16hi_f32(r23) + bias4[3], bf16lo_f32(r23) + bias4[2]);
    r01 = b01; r23 = b23;
  }
  if (epilogue == DXB_EPILOGUE_GELU_TANH) {
    r01 = cvt_bf16x2(gelu_tanh(bf16hi_f32(r01)), gelu_tanh(bf16lo_f32(r01)));
    r23 = cvt_bf16x2(gelu_tanh(bf16hi_f32(r23)), gelu_tanh(bf16lo_f32(r23)));
  }
  return make_uint2(r01, r23);
}

// MULTI: more than one token block (M > 128); a tile is then a (token block, column tile)
// pair.  The single-block kernel carries none of that bookkeeping.
// RELAID (int4 only): the packed bytes were rewritten by wq_relayout_w4_kernel so that one
// 32-bit word holds the k-pairs the TMEM store wants (see there); saves the byte permutes.
// MODE: the same pipeline compiled three times.  The two lean instances carry only what the
// common launches execute, which keeps their code a third of the general instance's: these
// launches last 8-15 us, and a kernel whose code is larger than the instruction cache pays for
// fetching it again in every launch (measured: 12.6 against 13.5 us on the headline shape).
//   kModeGeneral  every epilogue (activation, sum over ranks), tiles shared between CTAs
//                 through global partial sums, clusters
//   kModeWhole    whole tiles per CTA, plain epilogue (optional bias), no cluster
//   kModeCluster  one tile per cluster (K split, sum through distributed shared memory),
//                 plain epilogue
enum : int { kModeGeneral = 0, kModeWhole = 1, kModeCluster = 2 };

template <int BITS, bool HAS_ZERO, bool MULTI, bool RELAID, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
wq_gemm_tc(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_x,
           const WqParams p) {
  // A unit is 128 logical k of 128 weight columns in two planes of 64: for int4 the low and the
  // high nibbles of 64 packed rows (k and k + K/2), for int8 two consecutive blocks of 64 rows.
  constexpr int PLANES = 2;
  constexpr int A_STAGE_COLS = PLANES * 32;
  constexpr int UNIT_ROWS = BITS == 4 ? 64 : 128;   // packed rows per unit
  constexpr int W_STAGE = UNIT_ROWS * kTileN;       // bytes of one packed-weight stage

#ifdef DXB_TRACE
  const long long t_entry = clock64();
#endif
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[kNumBars];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
#ifdef DXB_TRACE
  __shared__ long long t_start;
#endif

  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t w_ring = smem0;
  const uint32_t x_ring = smem0 + p.w_stages * W_STAGE;
  const uint32_t bar0 = smem_u32(bars);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int SW = p.w_stages;

  // This CTA's contiguous range of (tile, unit) work.
  // Cluster mode: the `cluster` CTAs of one cluster share one tile, each taking a
  // contiguous slice of its K units; they add their partial sums through distributed
  // shared memory at the end (no global scratch, no counters).
  const int TU = p.total_units;
  const int G = static_cast<int>(gridDim.x);
  const int U = p.units_per_tile;
  constexpr bool kLean = MODE != kModeGeneral;
  const int C = MODE == kModeWhole ? 1 : p.cluster;  // kModeCluster is only launched with C > 1
  const bool clustered = MODE == kModeCluster || (MODE == kModeGeneral && C > 1);
  const bool tile_ranges = MODE == kModeWhole || (MODE == kModeGeneral && p.tile_ranges);
  // Ranges without a division on the way to the first weight load (a 64-bit division is a few
  // hundred cycles at the head of every launch): `range_q`, `range_r` are quotient and remainder
  // of what is being cut (a cluster's units by its size, or the tiles by the grid), so part i
  // starts at i * q + min(i, r).  Only unit ranges that cut tiles still divide.
  const int crank = clustered ? static_cast<int>(cluster_cta_rank()) : 0;
  const int ctile = clustered ? static_cast<int>(cluster_id_x()) : 0;
  const int part = clustered ? crank : static_cast<int>(blockIdx.x);
  const int cut_begin = part * p.range_q + (part < p.range_r ? part : p.range_r);
  const int cut_end = cut_begin + p.range_q + (part < p.range_r ? 1 : 0);
  const bool unit_ranges = MODE == kModeGeneral && !clustered && !tile_ranges;
  const int u_begin = clustered ? ctile * U + cut_begin
                      : !unit_ranges ? cut_begin * U : static_cast<int>(range_begin(blockIdx.x, TU, G));
  const int u_end = clustered ? ctile * U + cut_end
                    : !unit_ranges ? cut_end * U : static_cast<int>(range_begin(blockIdx.x + 1, TU, G));
  const int tile_begin = clustered ? ctile : !unit_ranges ? cut_begin : u_begin / U;
  const int ku_begin = clustered ? cut_begin : !unit_ranges ? 0 : u_begin - tile_begin * U;

  // Packed-weight producers (warps 0 and 3, alternate units): cursor of the next unit to load.
  // (Issuing the first loads before the CTA-wide set-up barrier, with the producers only
  // arriving at it, triggering the dependent launch earlier, staggering the teams' first
  // conversions, and a first conversion pass that only walks the code to fill the
  // instruction cache were all measured: none made the launch faster, so the plain order stays.)
  const int wp = warp == 0 ? 0 : 1;
  int w_u = u_begin + wp, w_tile = tile_begin, w_ku = ku_begin + wp, w_s = wp, w_ntile = 0;
  uint32_t w_ph = 0;
  auto w_issue = [&]() {
    if (elect_one()) {
      const uint32_t fw = bar0 + 8 * (kBarFullW + w_s);
      if (DX_DEBUG(2) && w_u >= u_begin + SW) {
        mbar_arrive(fw);  // experiment: reuse what the stage already holds
      } else {
        mbar_expect_tx(fw, W_STAGE);
        tma_load_2d(w_ring + w_s * W_STAGE, &tm_q, fw, (MULTI ? w_ntile : w_tile) * kTileN, w_ku * UNIT_ROWS);
      }
    }
    __syncwarp();
    w_u += 2;
    w_s += 2;
    if (w_s >= SW) { w_s -= SW; w_ph ^= 1u; }
    w_ku += 2;
    while (w_ku >= U) { w_ku -= U; ++w_tile; if (MULTI && ++w_ntile == p.tiles_n) w_ntile = 0; }
  };
  if (warp == 0 || warp == 3) {
    if (lane == 0) tma_prefetch_desc(&tm_q);
    // Each producer initialises the full and empty barriers of its own stages (even stages:
    // warp 0, odd: warp 3), the only ones it ever waits on, so it needs nobody else's set-up;
    // warp 3 also initialises the remaining barriers, which nobody touches before the set-up
    // barrier below.  Both clear the abort flag (same value) before anybody can wait.
    static_assert(kBarEmptyW - kBarFullW == 16 && kBarReady - kBarEmptyW == 16 && kNumBars - kBarReady <= 24,
                  "one lane per barrier below");
    if (lane < 8) {
      mbar_init(bar0 + 8 * (kBarFullW + wp + 2 * lane), bar_count(kBarFullW + wp + 2 * lane));
      mbar_init(bar0 + 8 * (kBarEmptyW + wp + 2 * lane), bar_count(kBarEmptyW + wp + 2 * lane));
    } else if (warp == 3 && kBarReady + lane - 8 < kNumBars) {
      mbar_init(bar0 + 8 * (kBarReady + lane - 8), bar_count(kBarReady + lane - 8));
    }
    if (lane == 0) {
      abort_flag = 0;
#ifdef DXB_TRACE
      if (warp == 3) {
        t_start = t_entry;  // trace builds: every stamp counts from the thread's first instruction
        DX_TRACE(5, 0);     // barriers initialised
      }
#endif
    }
    mbar_init_fence();
    __syncwarp();
    while (w_ku >= U) { w_ku -= U; ++w_tile; }
    w_ntile = MULTI ? w_tile % p.tiles_n : 0;
  } else if (warp == 2 && lane == 0) {
    tma_prefetch_desc(&tm_x);
  } else if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem0 = tmem_base_s;
  if (threadIdx.x == 0) DX_TRACE(5, 1);  // set-up barrier passed
  // The next kernel of the stream may start now: its weight loads and conversion do not
  // depend on this kernel; it waits (pdl_wait) before it touches activations or outputs.
  pdl_launch_dependents();

  volatile int* abortp = &abort_flag;

  // Cluster mode: send this CTA's fp32 partial rows from accumulator `d_tmem` (already
  // offset to the calling warp's lane quadrant) to their owners' receive buffers.
  auto cluster_send = [&](uint32_t d_tmem, int c, int n_local, int m_rows, int wk, int nwk) {
    const uint32_t recv0 = smem0 + static_cast<uint32_t>(p.recv_off);
    for (int c0 = 16 * wk; c0 < p.NU; c0 += 16 * nwk) {
      uint32_t ra[8], rb[8];
      tmem_ld_16x128b_x4(d_tmem + c0, ra);
      tmem_ld_16x128b_x4(d_tmem + (16u << 16) + c0, rb);
      tc_wait_ld();
      if (threadIdx.x == 0) DX_TRACE(7, 7);  // accumulator chunk in registers
#pragma unroll
      for (int rep = 0; rep < 4; ++rep) {
        const int m = c0 + 4 * rep + c;
        if (m < m_rows) {
          const int owner = (m * p.rows_inv) >> 16;
          const int row = crank * p.rows_per + (m - owner * p.rows_per);
          st_dsmem_b32x4(dsmem_addr(recv0 + static_cast<uint32_t>(row * kTileN + n_local) * 4u, owner),
                         ra[2 * rep], ra[2 * rep + 1], rb[2 * rep], rb[2 * rep + 1]);
        }
      }
    }
  };

  // ------------------------------------------------------------------ epilogue of one segment
  // A segment = this CTA's units of one tile, summed in accumulator `b`; run by the four
  // epilogue warps (one per TMEM lane quadrant).  Accumulator lane 32q + 8b + g holds weight
  // column 32q + 4g + b (see the dequant mapping), so the 16x128b load shape hands thread
  // (g, c) the four consecutive columns 4g..4g+3 of token 4*rep + c: one 8-byte store each.
  // Returns false when a bounded wait ran out.  (Letting the then idle dequant warps share
  // the last segment's columns was measured: it shortens a whole tile's epilogue by 0.3 us
  // but its register cost slows the cluster-split launches by more.)
  // Bias of this thread's four columns of a tile (fetched before waiting for the accumulator,
  // so that its latency is not added to the tail of the tile).
  auto load_bias4 = [&](int tile, float (&bias4)[4]) {
    const int ntile = MULTI ? tile % p.tiles_n : tile;
    const int n = ntile * kTileN + 32 * (warp & 3) + 4 * (lane >> 2);
    bias4[0] = bias4[1] = bias4[2] = bias4[3] = 0.f;
    if (p.bias != nullptr && n < p.N) {
      const uint2 bb = __ldg(reinterpret_cast<const uint2*>(p.bias + n));
      bias4[0] = bf16lo_f32(bb.x); bias4[1] = bf16hi_f32(bb.x);
      bias4[2] = bf16lo_f32(bb.y); bias4[3] = bf16hi_f32(bb.y);
    }
  };
  auto epilogue_segment = [&](int tile, int ku0, int nun, int b, const float (&bias4)[4]) -> bool {
    constexpr int wk = 0, nwk = 1, nthr = kEpilogueThreads;  // the four epilogue warps, all columns
    const int wtid = (warp - 4) * 32 + lane;
    const int q = warp & 3;
    const int c = lane & 3;
    const int g = lane >> 2;
    const int n_local = 32 * q + 4 * g;
    const bool has_bias = p.bias != nullptr;
    const bool whole = MODE == kModeWhole || (MODE == kModeGeneral && nun == U);
    const int tblock = MULTI ? tile / p.tiles_n : 0;  // token block of this tile
    const int ntile = tile - tblock * p.tiles_n;      // its 128 weight columns
    const int row0 = tblock * 128;
    const int m_rows = MULTI ? ((p.M - row0) < 128 ? (p.M - row0) : 128) : p.M;  // token rows in this block
    const int n = ntile * kTileN + n_local;
    const bool n_ok = n < p.N;
    // Sum over ranks fused into this launch (one token block only): finished rows go to
    // every rank's receive buffer instead of `out`; fused_finish then completes the tile.
    const bool fused = !kLean && p.peer.world > 1;
    const bool plain = kLean || (!fused && p.epilogue == DXB_EPILOGUE_NONE);
    const unsigned parity =
        fused ? (__ldcg(reinterpret_cast<const unsigned*>(p.peer.region[p.peer.rank])) & 1u) : 0u;
    auto fused_finish = [&]() -> bool {
      // The barrier orders every participant's peer stores before the signalling threads;
      // their release at system scope is cumulative, so it covers all of them (a system
      // fence costs about 1.7 us on this machine: one per rank to signal, not one per thread).
      named_bar_sync(1, nthr);
      if (wtid < p.peer.world) {
        fused_signal(p.peer, ntile, wtid, static_cast<unsigned>(m_rows));
        fused_wait(p.peer, ntile, wtid, static_cast<unsigned>(m_rows), abortp);
      }
      named_bar_sync(1, nthr);
      if (*abortp) return false;
      const int c4 = (wtid & 31) * 4;
      const int nn = ntile * kTileN + c4;
      if (nn < p.N) {
        float b4[4] = {0.f, 0.f, 0.f, 0.f};
        if (has_bias) {
          const uint2 bb = __ldg(reinterpret_cast<const uint2*>(p.bias + nn));
          b4[0] = bf16lo_f32(bb.x); b4[1] = bf16hi_f32(bb.x);
          b4[2] = bf16lo_f32(bb.y); b4[3] = bf16hi_f32(bb.y);
        }
        for (int m = wtid >> 5; m < m_rows; m += nthr >> 5) {
          const float4 a = fused_sum4(p.peer, parity, static_cast<long long>(m) * p.N + nn);
          *reinterpret_cast<uint2*>(p.out + static_cast<long long>(m) * p.ldo + nn) =
              finish_row4(a.x, a.y, a.z, a.w, b4, has_bias, p.epilogue);
        }
      }
      return true;
    };
    const uint32_t d_tmem = tmem_addr(tmem0 + b * p.NU, 32 * q, 0);
    if (whole) {
      for (int c0 = 16 * wk; c0 < p.NU; c0 += 16 * nwk) {
        uint32_t ra[8], rb[8];
        tmem_ld_16x128b_x4(d_tmem + c0, ra);
        tmem_ld_16x128b_x4(d_tmem + (16u << 16) + c0, rb);
        tc_wait_ld();
#pragma unroll
        for (int rep = 0; rep < 4; ++rep) {
          const int m = c0 + 4 * rep + c;
          if (n_ok && m < m_rows) {
            const float f0 = __uint_as_float(ra[2 * rep]), f1 = __uint_as_float(ra[2 * rep + 1]);
            const float f2 = __uint_as_float(rb[2 * rep]), f3 = __uint_as_float(rb[2 * rep + 1]);
            uint2* dst = reinterpret_cast<uint2*>(p.out + static_cast<long long>(row0 + m) * p.ldo + n);
            if (plain) {  // the common case, kept free of the optional epilogues' code
              uint2 pk;
              if (has_bias) {
                // Reference order: round the matmul to bf16, then add the bias in bf16.
                const uint32_t r01 = cvt_bf16x2(f1, f0), r23 = cvt_bf16x2(f3, f2);
                pk.x = cvt_bf16x2(bf16hi_f32(r01) + bias4[1], bf16lo_f32(r01) + bias4[0]);
                pk.y = cvt_bf16x2(bf16hi_f32(r23) + bias4[3], bf16lo_f32(r23) + bias4[2]);
              } else {
                pk.x = cvt_bf16x2(f1, f0);
                pk.y = cvt_bf16x2(f3, f2);
              }
              *dst = pk;
            } else if (fused) {
              fused_push4(p.peer, parity, static_cast<long long>(m) * p.N + n, f0, f1, f2, f3);
            } else {
              *dst = finish_row4(f0, f1, f2, f3, bias4, has_bias, p.epilogue);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && wk == 0) mbar_arrive(bar0 + 8 * (kBarAccEmpty + b));
      if (fused && !fused_finish()) return false;
    } else if (clustered) {
      // Cluster mode: CTA r of the cluster finishes token rows [r*rows_per, (r+1)*rows_per)
      // of the tile.  Every CTA sends each owner its fp32 partial rows straight from the
      // accumulator registers into the owner's receive buffer `crank` (distributed shared
      // memory stores); one cluster barrier later the owner only reads its own memory.
      // A cluster CTA has exactly this one segment, in accumulator 0, at the very end of its
      // work, when every other warp is idle: the accumulator stays where it is and ALL warps
      // send it after the CTA-wide barrier below (six warps per TMEM lane quadrant, 16
      // token columns each, instead of the four epilogue warps walking all of them).
    } else if (!kLean) {
      // A tile shared by several CTAs (equal unit ranges cut it): the CTA that holds the
      // tile's first units finishes it.  Ranges are contiguous and worked through in
      // order, so a CTA contributes to a tile it does not finish as its FIRST segment
      // and finishes a shared tile as its LAST one: by then the contributions have
      // normally been waiting in global scratch for a while, and the finisher only adds
      // them to its own accumulator (own sum first, then the slots in CTA order: the
      // result does not depend on timing).
      const int c_first = owner_of(static_cast<long long>(tile) * U, TU, G);
      const int c_last = owner_of(static_cast<long long>(tile) * U + U - 1, TU, G);
      const long long slot_elems = static_cast<long long>(p.NU) * kTileN;
      float* tile_ws = p.partials + static_cast<long long>(tile) * p.max_slots * slot_elems;
      if (ku0 > 0) {
        // contributor: park the fp32 sums, publish, carry on
        float* ws = tile_ws + (static_cast<int>(blockIdx.x) - c_first - 1) * slot_elems;
        for (int c0 = 16 * wk; c0 < p.NU; c0 += 16 * nwk) {
          uint32_t ra[8], rb[8];
          tmem_ld_16x128b_x4(d_tmem + c0, ra);
          tmem_ld_16x128b_x4(d_tmem + (16u << 16) + c0, rb);
          tc_wait_ld();
#pragma unroll
          for (int rep = 0; rep < 4; ++rep) {
            const int m = c0 + 4 * rep + c;
            if (m < m_rows)
              __stcg(reinterpret_cast<float4*>(ws + m * kTileN + n_local),
                     make_float4(__uint_as_float(ra[2 * rep]), __uint_as_float(ra[2 * rep + 1]),
                                 __uint_as_float(rb[2 * rep]), __uint_as_float(rb[2 * rep + 1])));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && wk == 0) mbar_arrive(bar0 + 8 * (kBarAccEmpty + b));
        __threadfence();
        named_bar_sync(1, nthr);
        if (wtid == 0) atomicAdd(&p.counters[tile], 1);
      } else {
        // finisher: wait (bounded) until every contributor has published
        const int ncontrib = c_last - c_first;
        if (wtid == 0) {
          if (wait_flag_ge(&p.counters[tile], ncontrib, abortp))
            p.counters[tile] = 0;  // ready for the next launch / graph replay
        }
        named_bar_sync(1, nthr);
        if (*abortp) return false;
        for (int c0 = 16 * wk; c0 < p.NU; c0 += 16 * nwk) {
          float4 v[4];
#pragma unroll
          for (int rep = 0; rep < 4; ++rep) v[rep] = make_float4(0.f, 0.f, 0.f, 0.f);
          // contributions in CTA order; the loads of one slot are in flight together
          for (int sl = 0; sl < ncontrib; ++sl) {
            float4 t4[4];
#pragma unroll
            for (int rep = 0; rep < 4; ++rep) {
              const int m = c0 + 4 * rep + c;
              t4[rep] = m < m_rows ? __ldcg(reinterpret_cast<const float4*>(
                                         tile_ws + sl * slot_elems + m * kTileN + n_local))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int rep = 0; rep < 4; ++rep) {
              if (sl == 0) {
                v[rep] = t4[rep];
              } else {
                v[rep].x += t4[rep].x; v[rep].y += t4[rep].y;
                v[rep].z += t4[rep].z; v[rep].w += t4[rep].w;
              }
            }
          }
          uint32_t ra[8], rb[8];
          tmem_ld_16x128b_x4(d_tmem + c0, ra);
          tmem_ld_16x128b_x4(d_tmem + (16u << 16) + c0, rb);
          tc_wait_ld();
#pragma unroll
          for (int rep = 0; rep < 4; ++rep) {
            const int m = c0 + 4 * rep + c;
            if (n_ok && m < m_rows) {
              const float f0 = __uint_as_float(ra[2 * rep]) + v[rep].x, f1 = __uint_as_float(ra[2 * rep + 1]) + v[rep].y;
              const float f2 = __uint_as_float(rb[2 * rep]) + v[rep].z, f3 = __uint_as_float(rb[2 * rep + 1]) + v[rep].w;
              if (fused)
                fused_push4(p.peer, parity, static_cast<long long>(m) * p.N + n, f0, f1, f2, f3);
              else
                *reinterpret_cast<uint2*>(p.out + static_cast<long long>(row0 + m) * p.ldo + n) =
                    finish_row4(f0, f1, f2, f3, bias4, has_bias, p.epilogue);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && wk == 0) mbar_arrive(bar0 + 8 * (kBarAccEmpty + b));
        if (fused && !fused_finish()) return false;
      }
    }
    return true;
  };

  if (warp == 0 || warp == 3) {
    // ============================================ TMA producer: packed weights
    // Two producer warps (0 and 3) take alternate units, which doubles the issue rate.
    // The whole warp runs the loop (so addresses and coordinates stay in uniform
    // registers, which the TMA instruction wants); one elected lane issues.
    {
      bool ok = true;
      // first pass over the ring: every stage is free
      for (int first = 0; first < (SW >> 1) && w_u < u_end; ++first) {
        w_issue();
        if (warp == 0 && lane == 0 && first == 0) DX_TRACE(5, 2);  // first weight load issued
      }
      while (w_u < u_end) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar0 + 8 * (kBarEmptyW + w_s), w_ph ^ 1u, abortp));
        if (!ok) break;
        w_issue();
      }
      if (!ok && lane == 0) {
        // Leaving early: let the copies already issued land before the CTA exits.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ============================================== TMA producer: activations
    // Activations may be the output of the previous kernel in the stream.
    pdl_wait();
    if (lane == 0) DX_TRACE(5, 3);  // the previous kernel of the stream is complete
    {
      int ku = ku_begin, t = 0;
      int ntile = MULTI ? tile_begin % p.tiles_n : 0;
      int row0 = MULTI ? (tile_begin / p.tiles_n) * 128 : 0;  // first token row of the token block
      uint32_t ph = 0;
      int issued = 0;
      bool ok = true;
      const uint32_t x_bytes = p.x_stage_bytes;
      for (int u = u_begin; u < u_end; ++u) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar0 + 8 * (kBarFree + t), ph ^ 1u, abortp));
        if (!ok) break;
        if (elect_one()) {
          const uint32_t rb = bar0 + 8 * (kBarReady + t);
          if (DX_DEBUG(1) && u >= u_begin + kAStages) {
            mbar_arrive(rb);  // experiment: reuse what the slot already holds
          } else {
          mbar_expect_tx(rb, x_bytes);
          if (BITS == 4) {
            tma_load_3d(x_ring + t * p.x_stage_bytes, &tm_x, rb, ku * 64, row0, 0);
          } else {  // two k-blocks of 64, one per plane
            tma_load_2d(x_ring + t * p.x_stage_bytes, &tm_x, rb, ku * 128, row0);
            tma_load_2d(x_ring + t * p.x_stage_bytes + (x_bytes >> 1), &tm_x, rb, ku * 128 + 64, row0);
          }
          }
        }
        __syncwarp();
        ++issued;
        if (++t == kAStages) { t = 0; ph ^= 1u; }
        if (++ku == U) {
          ku = 0;
          if (MULTI && ++ntile == p.tiles_n) { ntile = 0; row0 += 128; }
        }
      }
      if (!ok && lane == 0) {
        // Leaving early: give copies already issued time to land before the CTA exits.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
      }
      (void)issued;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ======================================================= MMA issuer ====
    // Warp-uniform loop as well: descriptors, TMEM addresses and barrier addresses
    // live in uniform registers; one elected lane issues the MMAs and commits.
    {
      const uint32_t idesc = idesc_bf16_f32(kTileN, p.NU);
      const uint64_t xdesc0 = smem_desc_kmajor_sw128(x_ring);
      const uint32_t x_stage16 = static_cast<uint32_t>(p.x_stage_bytes) >> 4;
      const uint32_t plane16 = static_cast<uint32_t>(p.NU * 128) >> 4;
      int t = 0, b = 0;
      uint32_t ph = 0, accph = 0;
      uint64_t xd = xdesc0;
      uint32_t a_tmem = tmem0 + kACol0;
      bool ok = true;
      int u = u_begin, ku0 = ku_begin, done = 0;
      const bool leader = elect_one();  // the one lane that issues; fixed for the whole loop
      while (u < u_end && ok) {
        const int left = u_end - u;
        const int nun = left < (U - ku0) ? left : (U - ku0);
        ok = __all_sync(0xffffffffu, mbar_wait(bar0 + 8 * (kBarAccEmpty + b), accph ^ 1u, abortp));
        if (!ok) break;
        const uint32_t d_tmem = tmem0 + b * p.NU;
        uint32_t accumulate = 0;
        for (int i = 0; i < nun; ++i) {
          if (!mbar_wait(bar0 + 8 * (kBarReady + t), ph, abortp)) { ok = false; break; }
          tc_fence_after();
          if (lane == 0 && done == 0) DX_TRACE(5, 4);  // first unit ready (weights in TMEM, activations in smem)
          if (leader && DX_DEBUG(32)) {
            // experiment: the two planes accumulate into different accumulators, alternating
            const uint32_t d2 = tmem0 + (b ^ 1) * p.NU;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              mma_ts(d_tmem, a_tmem + kk * 8, xd + kk * 2, idesc, kk == 0 ? accumulate : 1u);
              mma_ts(d2, a_tmem + 32 + kk * 8, xd + plane16 + kk * 2, idesc, kk == 0 ? accumulate : 1u);
            }
            tc_commit(bar0 + 8 * (kBarFree + t));
          } else if (leader && !DX_DEBUG(8)) {
            mma_ts(d_tmem, a_tmem, xd, idesc, accumulate);
#pragma unroll
            for (int kk = 1; kk < 4; ++kk) mma_ts(d_tmem, a_tmem + kk * 8, xd + kk * 2, idesc, 1u);
            if (PLANES == 2) {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                mma_ts(d_tmem, a_tmem + 32 + kk * 8, xd + plane16 + kk * 2, idesc, 1u);
            }
            tc_commit(bar0 + 8 * (kBarFree + t));
          } else if (leader) {
            tc_commit(bar0 + 8 * (kBarFree + t));
          }
          accumulate = 1;
          if (lane == 0) DX_TRACE(3, done);
          ++done;
          xd += x_stage16;
          a_tmem += A_STAGE_COLS;
          if (++t == kAStages) { t = 0; ph ^= 1u; xd = xdesc0; a_tmem = tmem0 + kACol0; }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (leader) tc_commit(bar0 + 8 * (kBarAccFull + b));
        u += nun;
        ku0 = 0;
        if (++b == 2) { b = 0; accph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // ========================================================= epilogue ====
    pdl_wait();  // outputs / scratch may still be in use by the previous kernel
    const int etid = (warp - 4) * 32 + lane;
    int b = 0;
    uint32_t accph = 0;
    int u = u_begin, ku0 = ku_begin, tile = tile_begin;
    while (u < u_end) {
      const int left = u_end - u;
      const int nun = left < (U - ku0) ? left : (U - ku0);
      float bias4[4];
      load_bias4(tile, bias4);
      if (!mbar_wait(bar0 + 8 * (kBarAccFull + b), accph, abortp)) break;
      if (etid == 0) DX_TRACE(0, tile - tile_begin);
      tc_fence_after();
      if (!epilogue_segment(tile, ku0, nun, b, bias4)) break;
      if (etid == 0) DX_TRACE(1, tile - tile_begin);
      u += nun;
      ku0 = 0;
      ++tile;
      if (++b == 2) { b = 0; accph ^= 1u; }
    }
  } else if (warp >= 8) {
    // ========================================================== dequant ====
    // Four teams of four warps; team j converts units j, j+4, j+8, ... of this CTA
    // into TMEM ring stage j, so four units are in flight and the per-unit chain
    // (barrier wake-up, shared-memory loads, TMEM store drain) of one team is
    // hidden behind the other three.
    // Thread (c = lane % 4, g = lane / 4) of quadrant q reads, for each slab of 8
    // packed rows, the 32-bit words at rows 2c and 2c+1, byte columns
    // 32q + 4g .. +3.  Byte b of the word is weight column 32q + 4g + b and goes to
    // TMEM lane 32q + 8b + g; rows (2c, 2c+1) form one bf16 pair = TMEM column c of
    // that slab: exactly the register layout of tcgen05.st.16x128b.
    const int team = (warp - 8) >> 2;
    const int q = warp & 3;
    const int c = lane & 3;
    const int g = lane >> 2;
    const uint32_t chunk = 2 * q + (g >> 2);
    const uint32_t off0 = (2 * c) * 128 + ((chunk ^ (2 * c)) << 4) + 4 * (g & 3);
    const uint32_t off1 = (2 * c + 1) * 128 + ((chunk ^ (2 * c + 1)) << 4) + 4 * (g & 3);
    const uint32_t lane_base = 32 * q;
    const int n_local = 32 * q + 4 * g;
    const int group_units = p.group / 64;   // quantisation group in planes of 64 k
    const int half_units = p.half_k / 64;    // int4: planes between the low and the high nibbles
    const uint2* sc_ptr = reinterpret_cast<const uint2*>(p.scales);
    const uint2* zr_ptr = reinterpret_cast<const uint2*>(p.zeros);
    const uint32_t a_tmem = tmem0 + kACol0 + team * A_STAGE_COLS;
    const uint32_t a_full_bar = bar0 + 8 * (kBarReady + team);
    const uint32_t a_empty_bar = bar0 + 8 * (kBarFree + team);

    // cursor of this team's current unit
    int u = u_begin + team;
    int tile = tile_begin, ku = ku_begin + team;
    while (ku >= U) { ku -= U; ++tile; }
    int ntile = MULTI ? tile % p.tiles_n : 0;  // column tile of `tile`, kept in step without divisions
    int s = team;  // SW is a multiple of the team count: stages j, j+4, ... belong to team j
    uint32_t ph = 0;
    uint32_t aph = 0;
    bool ok = true;
    // Scales / zero points come straight from global memory (they are tiny and stay in
    // L2), fetched one team-unit ahead so the load latency is never waited for.
    uint2 sc[PLANES], zr[PLANES], sc_nx[PLANES], zr_nx[PLANES];
    const int n4_stride = p.N >> 2;  // uint2 (4 x bf16) elements per scale row
    auto load_sz = [&](int tile_, int ntile_, int ku_, uint2 (&s_out)[PLANES], uint2 (&z_out)[PLANES]) {
      const int n = ntile_ * kTileN + n_local;
      const bool in = n < p.N && tile_ < p.tiles;
#pragma unroll
      for (int pl = 0; pl < PLANES; ++pl) {
        const int kunit = BITS == 4 ? ku_ + pl * half_units : 2 * ku_ + pl;  // plane of 64 k
        const int grp = p.group_shift >= 0 ? (kunit >> p.group_shift) : (kunit / group_units);
        const int idx = grp * n4_stride + (n >> 2);
        s_out[pl] = in ? __ldg(sc_ptr + idx) : make_uint2(0u, 0u);
        if (HAS_ZERO) z_out[pl] = in ? __ldg(zr_ptr + idx) : make_uint2(0u, 0u);
      }
    };
    if (u < u_end) load_sz(tile, MULTI ? ntile : tile, ku, sc_nx, zr_nx);
    while (u < u_end) {
#pragma unroll
      for (int pl = 0; pl < PLANES; ++pl) { sc[pl] = sc_nx[pl]; if (HAS_ZERO) zr[pl] = zr_nx[pl]; }
      {
        int ku_n = ku + kAStages, tile_n = tile;
        int ntile_n = ntile;
        while (ku_n >= U) { ku_n -= U; ++tile_n; if (MULTI && ++ntile_n == p.tiles_n) ntile_n = 0; }
        if (u + kAStages < u_end) load_sz(tile_n, MULTI ? ntile_n : tile_n, ku_n, sc_nx, zr_nx);
      }
      ok = mbar_wait(bar0 + 8 * (kBarFullW + s), ph, abortp);
      if (!ok) break;
      if (q == 0 && lane == 0) DX_TRACE(4, (u - u_begin));
      const uint32_t wsrc = w_ring + s * W_STAGE;
      uint32_t w0[8], w1[8];
#pragma unroll
      for (int sl = 0; sl < 8; ++sl) {
        w0[sl] = lds32(wsrc + off0 + sl * 1024);
        w1[sl] = lds32(wsrc + off1 + sl * 1024);
      }
      if (BITS == 4) {  // (int8 reads the second half of its stage further down)
        __syncwarp();  // every lane has its words in registers
        if (lane == 0) mbar_arrive(bar0 + 8 * (kBarEmptyW + s));
      }
      ok = mbar_wait(a_empty_bar, aph ^ 1u, abortp);
      if (!ok) break;
      if (q == 0 && lane == 0) DX_TRACE(6, (u - u_begin));
      tc_fence_after();
      if (BITS == 4) {
#pragma unroll
        for (int pl = 0; pl < 2; ++pl) {
          const uint32_t s2[4] = {dup_lo(sc[pl].x), dup_hi(sc[pl].x), dup_lo(sc[pl].y),
                                  dup_hi(sc[pl].y)};
          uint32_t z2[4];
          if (HAS_ZERO) {
            z2[0] = dup_lo(zr[pl].x); z2[1] = dup_hi(zr[pl].x);
            z2[2] = dup_lo(zr[pl].y); z2[3] = dup_hi(zr[pl].y);
          } else {
            z2[0] = z2[1] = z2[2] = z2[3] = 0x43084308u;  // 128 + 8
          }
#pragma unroll
          for (int rh = 0; rh < 2; ++rh) {
            uint32_t ra[8], rb[8];
#pragma unroll
            for (int sl = 0; sl < 4; ++sl) {
              if (DX_DEBUG(4)) {
                ra[2 * sl] = w0[4 * rh + sl]; ra[2 * sl + 1] = w1[4 * rh + sl];
                rb[2 * sl] = w0[4 * rh + sl]; rb[2 * sl + 1] = w1[4 * rh + sl];
              } else if (RELAID) {
                // The word of the even row holds the low-nibble plane, the word of the odd
                // row the high-nibble plane: nibble b is byte column b of the even row,
                // nibble 4 + b the same column of the odd row, so masking with 0x000F000F
                // after a shift by 4b yields the k-pair of column b directly.
                const uint32_t W = pl == 0 ? w0[4 * rh + sl] : w1[4 * rh + sl];
                ra[2 * sl + 0] = deq4(W, z2[0], s2[0]);
                ra[2 * sl + 1] = deq4(W >> 4, z2[1], s2[1]);
                rb[2 * sl + 0] = deq4(W >> 8, z2[2], s2[2]);
                rb[2 * sl + 1] = deq4(W >> 12, z2[3], s2[3]);
              } else {
                const uint32_t P = prmt(w0[4 * rh + sl], w1[4 * rh + sl], 0x5410u) >> (4 * pl);
                const uint32_t Q = prmt(w0[4 * rh + sl], w1[4 * rh + sl], 0x7632u) >> (4 * pl);
                ra[2 * sl + 0] = deq4(P, z2[0], s2[0]);
                ra[2 * sl + 1] = deq4(P >> 8, z2[1], s2[1]);
                rb[2 * sl + 0] = deq4(Q, z2[2], s2[2]);
                rb[2 * sl + 1] = deq4(Q >> 8, z2[3], s2[3]);
              }
            }
            if (!DX_DEBUG(16)) {
              tmem_st_16x128b_x4(tmem_addr(a_tmem + pl * 32 + 16 * rh, lane_base, 0), ra);
              tmem_st_16x128b_x4(tmem_addr(a_tmem + pl * 32 + 16 * rh, lane_base + 16, 0), rb);
            } else {
              asm volatile("" ::"r"(ra[0] ^ ra[1] ^ ra[2] ^ ra[3] ^ ra[4] ^ ra[5] ^ ra[6] ^ ra[7] ^ rb[0] ^ rb[1] ^ rb[2] ^
                                    rb[3] ^ rb[4] ^ rb[5] ^ rb[6] ^ rb[7]));  // keep the conversion alive
            }
          }
        }
      } else {
#pragma unroll
        for (int pl = 0; pl < 2; ++pl) {
          if (pl == 1) {
            // rows 64..127 of the unit; after these loads the stage can be refilled
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) {
              w0[sl] = lds32(wsrc + 8192 + off0 + sl * 1024);
              w1[sl] = lds32(wsrc + 8192 + off1 + sl * 1024);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar0 + 8 * (kBarEmptyW + s));
          }
          const float sf[4] = {bf16lo_f32(sc[pl].x), bf16hi_f32(sc[pl].x), bf16lo_f32(sc[pl].y),
                               bf16hi_f32(sc[pl].y)};
          float cz[4];
          if (HAS_ZERO) {
            cz[0] = 8388608.0f + bf16lo_f32(zr[pl].x); cz[1] = 8388608.0f + bf16hi_f32(zr[pl].x);
            cz[2] = 8388608.0f + bf16lo_f32(zr[pl].y); cz[3] = 8388608.0f + bf16hi_f32(zr[pl].y);
          } else {
            cz[0] = cz[1] = cz[2] = cz[3] = 8388608.0f + 128.0f;
          }
#pragma unroll
          for (int rh = 0; rh < 2; ++rh) {
            uint32_t ra[8], rb[8];
#pragma unroll
            for (int sl = 0; sl < 4; ++sl) {
              const uint32_t x0 = w0[4 * rh + sl], x1 = w1[4 * rh + sl];
              ra[2 * sl + 0] = cvt_bf16x2(deq8(x1, 0, cz[0], sf[0]), deq8(x0, 0, cz[0], sf[0]));
              ra[2 * sl + 1] = cvt_bf16x2(deq8(x1, 1, cz[1], sf[1]), deq8(x0, 1, cz[1], sf[1]));
              rb[2 * sl + 0] = cvt_bf16x2(deq8(x1, 2, cz[2], sf[2]), deq8(x0, 2, cz[2], sf[2]));
              rb[2 * sl + 1] = cvt_bf16x2(deq8(x1, 3, cz[3], sf[3]), deq8(x0, 3, cz[3], sf[3]));
            }
            tmem_st_16x128b_x4(tmem_addr(a_tmem + pl * 32 + 16 * rh, lane_base, 0), ra);
            tmem_st_16x128b_x4(tmem_addr(a_tmem + pl * 32 + 16 * rh, lane_base + 16, 0), rb);
          }
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_full_bar);
      if (q == 0 && lane == 0) DX_TRACE(2, (u - u_begin));
      aph ^= 1u;
      s += kAStages;
      if (s >= SW) { s -= SW; ph ^= 1u; }
      ku += kAStages;
      while (ku >= U) { ku -= U; ++tile; if (MULTI && ++ntile == p.tiles_n) ntile = 0; }
      u += kAStages;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) DX_TRACE(7, 1);  // every role is through its loop
  if (clustered) {
    // The cluster's tile: token block and column tile.
    const int tblock = MULTI ? ctile / p.tiles_n : 0;
    const int ntile = ctile - tblock * p.tiles_n;
    const int row0 = tblock * 128;
    const int m_rows = MULTI ? ((p.M - row0) < 128 ? (p.M - row0) : 128) : p.M;
    const int m_lo = crank * p.rows_per;
    const int m_hi = (m_lo + p.rows_per) < m_rows ? (m_lo + p.rows_per) : m_rows;
    const uint32_t recv0 = smem0 + static_cast<uint32_t>(p.recv_off);
    const uint32_t src_stride = static_cast<uint32_t>(p.rows_per * kTileN) * 4u;
    const bool has_bias = p.bias != nullptr;
    // Every item of one thread has the same four columns (kThreads is a multiple of 32):
    // their bias is fetched before the barrier, off the critical path.
    const int c4 = (threadIdx.x & 31) * 4;
    const int n = ntile * kTileN + c4;
    float bias4[4] = {0.f, 0.f, 0.f, 0.f};
    if (has_bias && n < p.N) {
      const uint2 bb = __ldg(reinterpret_cast<const uint2*>(p.bias + n));
      bias4[0] = bf16lo_f32(bb.x); bias4[1] = bf16hi_f32(bb.x);
      bias4[2] = bf16lo_f32(bb.y); bias4[3] = bf16hi_f32(bb.y);
    }
    if (p.recv_alias) {
      // The receive buffers lie over the rings, which the peers may still be using.  Every
      // CTA of the cluster is past its main loop after this barrier: nothing reads or writes
      // the rings any more, so the buffers may be filled.
      cluster_sync_all();
    }
    // The epilogue warps have seen the accumulator complete before the CTA-wide barrier above.
    tc_fence_after();
    if (threadIdx.x == 0) DX_TRACE(7, 6);  // about to send
    cluster_send(tmem_addr(tmem0, 32 * (warp & 3), 0), lane & 3, 32 * (warp & 3) + 4 * (lane >> 2), m_rows,
                 warp >> 2, kThreads / 128);
    tc_fence_before();
    if (threadIdx.x == 0) DX_TRACE(7, 2);  // partial sums sent
    // After this barrier every partial row of this CTA's share has arrived in its receive
    // buffers: sum them in rank order (deterministic), add the bias, write bf16.  Nothing
    // remote is touched any more, so CTAs leave independently.
    cluster_sync_all();
    if (threadIdx.x == 0) DX_TRACE(7, 3);  // cluster barrier passed
    pdl_wait();
    if (threadIdx.x == 0) DX_TRACE(7, 4);  // previous kernel complete
    const bool fused = !kLean && p.peer.world > 1;
    const int epi = kLean ? static_cast<int>(DXB_EPILOGUE_NONE) : p.epilogue;
    const unsigned parity =
        fused ? (__ldcg(reinterpret_cast<const unsigned*>(p.peer.region[p.peer.rank])) & 1u) : 0u;
    if (n < p.N) {
      for (int i = threadIdx.x; i < (m_hi - m_lo) * 32; i += kThreads) {
        const int j = i >> 5;
        const uint32_t a0 = recv0 + static_cast<uint32_t>(j * kTileN + c4) * 4u;
        float4 v[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          v[r] = r < C ? ld_smem_f4(a0 + r * src_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < 8; ++r) {  // rank order: the sum does not depend on timing
          acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
        }
        if (fused)
          fused_push4(p.peer, parity, static_cast<long long>(m_lo + j) * p.N + n, acc.x, acc.y, acc.z, acc.w);
        else
          *reinterpret_cast<uint2*>(p.out + static_cast<long long>(row0 + m_lo + j) * p.ldo + n) =
              finish_row4(acc.x, acc.y, acc.z, acc.w, bias4, has_bias, epi);
      }
    }
    if (threadIdx.x == 0) DX_TRACE(7, 5);  // rows summed and stored
    if (fused) {
      // This CTA's rows of the tile are on their way to every rank: publish them (the
      // barrier orders all stores before the signalling threads' cumulative release), wait
      // for the whole tile from every rank, then finish this CTA's rows from the local slots.
      __syncthreads();
      if (threadIdx.x < p.peer.world && m_hi > m_lo) {  // a CTA without rows has nothing to do
        fused_signal(p.peer, ntile, threadIdx.x, static_cast<unsigned>(m_hi - m_lo));
        fused_wait(p.peer, ntile, threadIdx.x, static_cast<unsigned>(m_rows), abortp);
      }
      __syncthreads();
      if (!abort_flag && n < p.N) {
        for (int i = threadIdx.x; i < (m_hi - m_lo) * 32; i += kThreads) {
          const int m = m_lo + (i >> 5);
          const float4 a = fused_sum4(p.peer, parity, static_cast<long long>(m) * p.N + n);
          *reinterpret_cast<uint2*>(p.out + static_cast<long long>(m) * p.ldo + n) =
              finish_row4(a.x, a.y, a.z, a.w, bias4, has_bias, epi);
        }
      }
    }
  }
  if (!kLean && p.peer.world > 1) {
    // The last CTA to leave moves the per-tile row baselines and the epoch on for the next
    // call (every other CTA has finished reading them by then).
    __shared__ int is_last;
    __syncthreads();
    unsigned char* mine = p.peer.region[p.peer.rank];
    unsigned* control = reinterpret_cast<unsigned*>(mine);
    if (threadIdx.x == 0) {
      __threadfence();
      is_last = atomicAdd(control + 1, 1u) == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (is_last) {
      __threadfence();
      for (int i = threadIdx.x; i < p.tiles_n * p.peer.world; i += kThreads) {
        unsigned* bp = fused_base(mine, i / p.peer.world, i % p.peer.world);
        *bp = __ldcg(bp) + static_cast<unsigned>(p.M);
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        control[1] = 0;
        control[0] = __ldcg(control) + 1;
      }
    }
  }
  if (threadIdx.x == 0) DX_TRACE(7, 0);
  if (warp == 1) tmem_dealloc(tmem0, 512);
  if (threadIdx.x == 0 && abort_flag) {
    pdl_wait();
    atomicExch(p.status, DXB_ERR_KERNEL_TIMEOUT);
  }
}

// ------------------------------------------------ load-time weight re-layout
// int4 only.  The reference packs byte [i, n] = row i (low nibble) | row i + K/2 (high
// nibble) (python/dexter/quant.py:62-72).  For every aligned block of 2 packed rows x 4
// byte columns (the two 32-bit words one dequant thread reads per slab of 8 rows) the 16
// nibbles are regrouped: the word at the even row keeps the low-nibble plane, the word at
// the odd row the high-nibble plane; inside a word, nibble b (bits 4b..4b+3) is byte column b
// of the even row and nibble 4 + b the same column of the odd row.  `(word >> 4b) &
// 0x000F000F` is then the bf16x2 mantissa pair (k, k+1) of column b: no byte permute.
// Same shape, same strides, same tiles; the transform is its own inverse pair (forward /
// inverse below) and is applied once per weight, never per call.
__device__ __forceinline__ uint32_t squeeze_nibbles(uint32_t v) {  // nibbles at bits 0,8,16,24 -> 0,4,8,12
  return (v & 0xFu) | ((v >> 4) & 0xF0u) | ((v >> 8) & 0xF00u) | ((v >> 12) & 0xF000u);
}
__device__ __forceinline__ uint32_t spread_nibbles(uint32_t h) {   // nibbles at bits 0,4,8,12 -> 0,8,16,24
  return (h & 0xFu) | ((h & 0xF0u) << 4) | ((h & 0xF00u) << 8) | ((h & 0xF000u) << 12);
}
__global__ void wq_relayout_w4_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                      long long row_pairs, int n4, int inverse) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= row_pairs * n4) return;
  const long long rp = idx / n4;
  const int j = static_cast<int>(idx - rp * n4);
  const long long i0 = (2 * rp) * n4 + j, i1 = (2 * rp + 1) * n4 + j;
  const uint32_t w0 = in[i0], w1 = in[i1];
  if (!inverse) {
    out[i0] = squeeze_nibbles(w0 & 0x0F0F0F0Fu) | (squeeze_nibbles(w1 & 0x0F0F0F0Fu) << 16);
    out[i1] = squeeze_nibbles((w0 >> 4) & 0x0F0F0F0Fu) | (squeeze_nibbles((w1 >> 4) & 0x0F0F0F0Fu) << 16);
  } else {
    out[i0] = spread_nibbles(w0 & 0xFFFFu) | (spread_nibbles(w1 & 0xFFFFu) << 4);
    out[i1] = spread_nibbles(w0 >> 16) | (spread_nibbles(w1 >> 16) << 4);
  }
}

// Value 0..15 of logical row k, column n of an int4 weight in either layout.
__device__ __forceinline__ uint32_t fetch_q4(const uint8_t* __restrict__ qw, int N, int half, int k, int n,
                                             int relaid) {
  const int plane = k < half ? 0 : 1;
  const int r = k - plane * half;  // packed row
  if (!relaid) return (qw[static_cast<long long>(r) * N + n] >> (4 * plane)) & 0xFu;
  const uint32_t word = reinterpret_cast<const uint32_t*>(qw)[(static_cast<long long>(r & ~1) + plane) * (N >> 2) + (n >> 2)];
  return (word >> (16 * (r & 1) + 4 * (n & 3))) & 0xFu;
}

// --------------------------------------------- dense dequantised weight dump
// W[k,n] bf16 with the same bit-pattern arithmetic as the tensor-core kernel;
// used to check the dequantisation bit for bit against the reference.
template <int BITS>
__global__ void wq_dequant_kernel(const uint8_t* __restrict__ qw, const __nv_bfloat16* __restrict__ scales,
                                  const __nv_bfloat16* __restrict__ zeros, __nv_bfloat16* __restrict__ out,
                                  int N, int K, int group, int relaid) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(K) * N;
  if (idx >= total) return;
  const int k = static_cast<int>(idx / N);
  const int n = static_cast<int>(idx % N);
  const int gi = k / group;
  const uint32_t sbits = __bfloat16_as_ushort(scales[static_cast<long long>(gi) * N + n]);
  if (BITS == 4) {
    const uint32_t byte = fetch_q4(qw, N, K / 2, k, n, relaid);
    const uint32_t z = zeros ? __bfloat16_as_ushort(zeros[static_cast<long long>(gi) * N + n]) : 0x4308u;
    const uint32_t r = deq4(byte, z | (z << 16), sbits | (sbits << 16));
    out[idx] = __ushort_as_bfloat16(static_cast<unsigned short>(r & 0xFFFFu));
  } else {
    const uint32_t byte = qw[idx];
    const float cz = 8388608.0f + (zeros ? __bfloat162float(zeros[static_cast<long long>(gi) * N + n]) : 128.0f);
    const float v = deq8(byte, 0, cz, __uint_as_float(sbits << 16));
    out[idx] = __ushort_as_bfloat16(static_cast<unsigned short>(cvt_bf16x2(0.0f, v) & 0xFFFFu));
  }
}

// ------------------------------------------------------ any-shape CUDA path
// Plain CUDA-core kernel for shapes the tensor-core kernel does not take (N not
// a multiple of 16, groups that are not a multiple of 64 rows, K/2 not a multiple
// of 64).  One thread per output column, 8 tokens per block row; slow but exact
// in the same sense (bit-identical W, fp32 accumulation).
template <int BITS>
__global__ void wq_gemm_simt(const __nv_bfloat16* __restrict__ x, long long ldx, const uint8_t* __restrict__ qw,
                             const __nv_bfloat16* __restrict__ scales, const __nv_bfloat16* __restrict__ zeros,
                             const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, long long ldo,
                             int M, int N, int K, int group, int relaid, int epilogue) {
  constexpr int MT = 8;
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int m0 = blockIdx.y * MT;
  if (n >= N) return;
  float acc[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i) acc[i] = 0.0f;
  const int half = K / 2;
  for (int k = 0; k < K; ++k) {
    const int gi = k / group;
    const uint32_t sbits = __bfloat16_as_ushort(scales[static_cast<long long>(gi) * N + n]);
    float w;
    if (BITS == 4) {
      const uint32_t byte = fetch_q4(qw, N, half, k, n, relaid);
      const uint32_t z = zeros ? __bfloat16_as_ushort(zeros[static_cast<long long>(gi) * N + n]) : 0x4308u;
      w = __uint_as_float(deq4(byte, z | (z << 16), sbits | (sbits << 16)) << 16);
    } else {
      const float cz = 8388608.0f + (zeros ? __bfloat162float(zeros[static_cast<long long>(gi) * N + n]) : 128.0f);
      const float v = deq8(qw[static_cast<long long>(k) * N + n], 0, cz, __uint_as_float(sbits << 16));
      w = __uint_as_float((cvt_bf16x2(0.0f, v) & 0xFFFFu) << 16);
    }
#pragma unroll
    for (int i = 0; i < MT; ++i)
      if (m0 + i < M) acc[i] += __bfloat162float(x[static_cast<long long>(m0 + i) * ldx + k]) * w;
  }
#pragma unroll
  for (int i = 0; i < MT; ++i)
    if (m0 + i < M) {
      __nv_bfloat16 o = __float2bfloat16_rn(acc[i]);
      if (bias) o = __float2bfloat16_rn(__bfloat162float(o) + __bfloat162float(bias[n]));
      if (epilogue == DXB_EPILOGUE_GELU_TANH) o = __float2bfloat16_rn(gelu_tanh(__bfloat162float(o)));
      out[static_cast<long long>(m0 + i) * ldo + n] = o;
    }
}

// ------------------------------------------------------------------ host side
static long long* g_trace = nullptr;

// Upper bound of the polled waits on flags that another GPU writes, in polls of about a
// quarter of a microsecond (default: about a second).
static std::atomic<unsigned> g_wait_tries{4000000u};
unsigned wait_tries() { return g_wait_tries.load(std::memory_order_relaxed); }

// Programmatic dependent launch is on unless DEXTER_B200_PDL=0.
static bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("DEXTER_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

// What a call asks for beyond the plain GEMM (dxb_gemm_opts, checked and copied).
struct Opts {
  int relaid = 0;
  int epilogue = DXB_EPILOGUE_NONE;
  int max_ctas = 0;
  int serialize = 0;
  PeerFuse peer = {};
};

struct Plan {
  int NU, planes, rows, unit_rows, w_stage_bytes, units_per_tile, tiles, tiles_n, total_units, stages,
      w_stages, x_stage_bytes, ctas,
      max_slots, nacc, recv_bytes, recv_off, recv_alias, whole;
  size_t smem_bytes;
};

// Cost, in units, of finishing a tile that equal unit ranges cut between CTAs: the finisher
// reads the other CTAs' fp32 partial tiles from L2 and adds them to its accumulator.
static int fixup_units(int NU) {
  static const int forced = [] {
    const char* e = getenv("DEXTER_B200_FIXUP_UNITS");
    return e ? atoi(e) : -1;
  }();
  if (forced >= 0) return forced;
  // measured: 83 x 3072 x 14336 takes 19 us with 148 equal ranges against 14 us with one tile
  // on each of 112 CTAs, i.e. finishing shared tiles costs about as much as 20 units
  return NU > 96 ? 32 : 20;
}

static Plan make_plan_uncached(int M, int N, int K, int bits, int sms, int max_ctas, bool allow_split) {
  Plan pl{};
  // More than 128 tokens: token blocks of 128, each (block, column tile) pair is a tile of
  // its own, so one launch covers all of them and every SM stays busy.
  const int blocks = (M + 127) / 128;
  pl.NU = blocks > 1 ? 128 : ((M + 15) / 16) * 16;
  // A unit is 128 logical k in two planes of 64: 64 packed rows of int4, 128 rows of int8.
  pl.planes = 2;
  pl.rows = bits == 4 ? K / 2 : K;
  pl.unit_rows = bits == 4 ? 64 : 128;
  pl.w_stage_bytes = pl.unit_rows * kTileN;
  pl.units_per_tile = pl.rows / pl.unit_rows;
  pl.tiles_n = (N + kTileN - 1) / kTileN;
  pl.tiles = pl.tiles_n * blocks;
  pl.total_units = pl.units_per_tile * pl.tiles;
  pl.x_stage_bytes = pl.planes * pl.NU * 128;
  // Shared memory: four activation stages (one per unit slot, like the TMEM ring) and
  // as deep a ring of packed-weight stages as still fits: those come from HBM and
  // need the most bytes in flight.  The depth is a multiple of four so that every
  // stage is only ever used by one dequant team, in order.
  pl.stages = kAStages;
  // Launches that may split tiles over a cluster keep room for its receive buffers
  // (at most NU + 8 token rows of 128 fp32) behind the two rings.
  const int budget_ctas = (max_ctas > 0 && max_ctas < sms) ? max_ctas : sms;
  pl.recv_bytes = (pl.tiles * 2 <= budget_ctas && pl.units_per_tile >= 2) ? (pl.NU + 8) * kTileN * 4 : 0;
  int w_stages = (kSmemBudget - pl.recv_bytes - kAStages * pl.x_stage_bytes) / pl.w_stage_bytes;
  pl.recv_alias = 0;
  if (pl.recv_bytes > 0 && (w_stages / kAStages) * kAStages * pl.w_stage_bytes < 2 * kAStages * kWStage) {
    // Not enough room for a useful weight ring next to the receive buffers (more than 96
    // tokens): let them lie over the rings instead.  The partial rows are then sent after
    // a cluster barrier at the end of the main loop, when the rings are idle.
    w_stages = (kSmemBudget - kAStages * pl.x_stage_bytes) / pl.w_stage_bytes;
    pl.recv_alias = 1;
  }
  w_stages = (w_stages / kAStages) * kAStages;
  if (w_stages > kMaxWStages) w_stages = kMaxWStages;
  pl.w_stages = w_stages;
  const int rings = pl.w_stages * pl.w_stage_bytes + pl.stages * pl.x_stage_bytes;
  if (pl.recv_alias && pl.recv_bytes > rings) {  // does not fit there either: no cluster split
    pl.recv_alias = 0;
    pl.recv_bytes = 0;
  }
  pl.recv_off = pl.recv_alias ? 0 : rings;
  pl.smem_bytes = static_cast<size_t>(rings) + (pl.recv_alias ? 0 : pl.recv_bytes) + 1024;
  // Grid: `budget` CTAs at most (all SMs unless the caller caps it, e.g. to run several
  // GEMMs side by side).
  const int budget = budget_ctas;
  // Two ways to hand out the work.  Whole tiles: every CTA takes `rounds` complete tiles
  // (CTAs may idle, nothing is split).  Equal unit ranges over all CTAs: nobody idles, but
  // the tiles cut by a range boundary are finished through global scratch (see the
  // epilogue).  Take whichever ends sooner.  (Few tiles in one token block are split over
  // clusters instead; the launcher decides that, see launch_tc.)
  const int rounds = (pl.tiles + budget - 1) / budget;
  const int whole_ctas = (pl.tiles + rounds - 1) / rounds;
  const long long whole_units = static_cast<long long>(rounds) * pl.units_per_tile;
  const long long split_units = (pl.total_units + budget - 1) / budget + fixup_units(pl.NU);
  // whole tiles: CTA c takes tiles [c * tiles / ctas, (c + 1) * tiles / ctas), at most `rounds`
  const bool whole = !allow_split || whole_units <= split_units;
  int ctas = whole ? whole_ctas : budget;
  if (ctas > pl.total_units) ctas = pl.total_units;
  pl.ctas = ctas;
  pl.whole = whole ? 1 : 0;
  pl.nacc = 2;
  int max_slots = 1;
  for (int t = 0; t < pl.tiles && !whole; ++t) {
    const long long u0 = static_cast<long long>(t) * pl.units_per_tile;
    const int c0 = owner_of(u0, pl.total_units, ctas);
    const int c1 = owner_of(u0 + pl.units_per_tile - 1, pl.total_units, ctas);
    if (c1 - c0 + 1 > max_slots) max_slots = c1 - c0 + 1;
  }
  pl.max_slots = max_slots;
  return pl;
}

// Plans only depend on the shape, so they are computed once per shape and thread.
static Plan make_plan(int M, int N, int K, int bits, int sms, int max_ctas, bool allow_split = true) {
  struct Key {
    int M, N, K, bits, sms, max_ctas, split;
    bool operator==(const Key& o) const {
      return M == o.M && N == o.N && K == o.K && bits == o.bits && sms == o.sms && max_ctas == o.max_ctas &&
             split == o.split;
    }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      size_t h = 1469598103934665603ull;
      for (int v : {k.M, k.N, k.K, k.bits, k.sms, k.max_ctas, k.split}) h = (h ^ static_cast<size_t>(v)) * 1099511628211ull;
      return h;
    }
  };
  static thread_local std::unordered_map<Key, Plan, Hash> cache;
  const Key key{M, N, K, bits, sms, max_ctas, allow_split ? 1 : 0};
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() > 4096) cache.clear();
  return cache.emplace(key, make_plan_uncached(M, N, K, bits, sms, max_ctas, allow_split)).first->second;
}

// The counter block has one fixed size so that calls with different tile counts
// never let one call's partial sums land on another call's counters.
static size_t counters_bytes(int) { return static_cast<size_t>(kMaxTiles) * 4; }

// Shapes wq_gemm_tc takes: those of tc_supported, and for int8 whole units of 128 rows.
static bool gemm_tc_supported(int M, int N, int K, int group, int bits) {
  return tc_supported(M, N, K, group, bits) && (bits != 8 || K % 128 == 0);
}

// Workspace the tensor-core launch of this problem needs (status, counters, partial sums).
static size_t plan_workspace_bytes(int M, int N, int K, int bits, int max_ctas) {
  DeviceInfo& di = device_info();
  const Plan pl = make_plan(M, N, K, bits, di.sms > 0 ? di.sms : 148, max_ctas);
  return kStatusBytes + counters_bytes(pl.tiles) +
         static_cast<size_t>(pl.tiles) * pl.max_slots * pl.NU * kTileN * sizeof(float);
}

// TMA tensor maps are encoded once per (pointer, geometry) and thread, not per call.
struct MapKey {
  const void* ptr;
  long long a, b, c;
  int kind;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && a == o.a && b == o.b && c == o.c && kind == o.kind; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr) * 1099511628211ull;
    for (long long v : {k.a, k.b, k.c, static_cast<long long>(k.kind)}) h = (h ^ static_cast<size_t>(v)) * 1099511628211ull;
    return h;
  }
};
template <class Encode>
static const CUtensorMap* cached_map(const MapKey& key, Encode&& encode) {
  static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  auto it = cache.find(key);
  if (it != cache.end()) return &it->second;
  if (cache.size() > 16384) cache.clear();
  CUtensorMap m;
  if (!encode(&m)) return nullptr;
  return &cache.emplace(key, m).first->second;
}

using TcKernel = void (*)(const CUtensorMap, const CUtensorMap, const WqParams);

template <int BITS, bool HAS_ZERO, bool MULTI, bool RELAID>
static TcKernel pick_mode(int mode) {
  switch (mode) {
    case kModeWhole: return wq_gemm_tc<BITS, HAS_ZERO, MULTI, RELAID, kModeWhole>;
    case kModeCluster: return wq_gemm_tc<BITS, HAS_ZERO, MULTI, RELAID, kModeCluster>;
    default: return wq_gemm_tc<BITS, HAS_ZERO, MULTI, RELAID, kModeGeneral>;
  }
}

template <int BITS, bool HAS_ZERO>
static TcKernel pick_kernel(bool multi, bool relaid, int mode) {
  if (BITS == 4 && relaid)
    return multi ? pick_mode<BITS, HAS_ZERO, true, BITS == 4>(mode) : pick_mode<BITS, HAS_ZERO, false, BITS == 4>(mode);
  return multi ? pick_mode<BITS, HAS_ZERO, true, false>(mode) : pick_mode<BITS, HAS_ZERO, false, false>(mode);
}

template <int BITS, bool HAS_ZERO>
static int launch_tc(const void* x, long long ldx, const void* qw, const void* scales,
                     const void* zeros, const void* bias, void* out, long long ldo, int M, int N,
                     int K, int group, void* workspace, size_t workspace_bytes, const Opts& opts,
                     cudaStream_t stream) {
  DeviceInfo& di = device_info();
  const int max_ctas = opts.max_ctas;
  Plan plan = make_plan(M, N, K, BITS, di.sms, max_ctas);
  const Plan* plp = &plan;
  if (plp->w_stages < kAStages) return DXB_ERR_UNSUPPORTED;
  // Status word and counters are always needed; the partial sums only if the launch ends up
  // splitting tiles through global scratch (checked below, once the cluster size is known).
  if (workspace == nullptr || workspace_bytes < kStatusBytes + counters_bytes(plp->tiles))
    return DXB_ERR_WORKSPACE;

  int dev = 0;
  cudaGetDevice(&dev);
  static thread_local int attr_dev = -1;
  if (attr_dev != dev) {
    bool ok = true;
    auto set = [&](auto kern) {
      ok = ok && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 1024) == cudaSuccess;
    };
    for (int multi = 0; multi < 2; ++multi)
      for (int relaid = 0; relaid < (BITS == 4 ? 2 : 1); ++relaid)
        for (int mode = 0; mode < 3; ++mode) set(pick_kernel<BITS, HAS_ZERO>(multi, relaid, mode));
    if (!ok) return DXB_ERR_CUDA;
    attr_dev = dev;
  }
  const bool multi = plp->tiles > plp->tiles_n;
  const bool relaid = BITS == 4 && opts.relaid;
  // The lean instances serve the plain epilogue; which of the two follows from the plan below.
  const bool lean = opts.epilogue == DXB_EPILOGUE_NONE && opts.peer.world <= 1;
  auto kernel = pick_kernel<BITS, HAS_ZERO>(multi, relaid, lean ? kModeCluster : kModeGeneral);

  // Few tiles: split each tile's K range over a thread-block cluster (<= 8 CTAs) that
  // reduces through distributed shared memory.  The cluster size is the largest one for
  // which all clusters are resident at once; the answer is cached per configuration.
  int cluster = 1;
  const int budget = (max_ctas > 0 && max_ctas < di.sms) ? max_ctas : di.sms;
  if (plp->recv_bytes > 0 && plp->tiles * 2 <= budget && plp->units_per_tile >= 2) {
    static thread_local std::unordered_map<long long, int> cache;
    const long long key = (static_cast<long long>(dev) << 48) ^ (static_cast<long long>(plp->tiles) << 28) ^
                          (static_cast<long long>(plp->units_per_tile) << 8) ^ static_cast<long long>(plp->NU >> 4) ^
                          (static_cast<long long>(budget) << 38) ^ (static_cast<long long>(multi) << 58) ^
                          (static_cast<long long>(relaid) << 59) ^ (static_cast<long long>(lean) << 60);
    auto it = cache.find(key);
    if (it != cache.end()) {
      cluster = it->second;
    } else {
      int cmax = budget / plp->tiles;
      if (cmax > 8) cmax = 8;
      if (cmax > plp->units_per_tile) cmax = plp->units_per_tile;
      for (int c = cmax; c >= 2; --c) {
        cudaLaunchConfig_t qcfg = {};
        qcfg.gridDim = dim3(plp->tiles * c);
        qcfg.blockDim = dim3(kThreads);
        qcfg.dynamicSmemBytes = plp->smem_bytes;
        cudaLaunchAttribute qattr[1];
        qattr[0].id = cudaLaunchAttributeClusterDimension;
        qattr[0].val.clusterDim.x = c;
        qattr[0].val.clusterDim.y = 1;
        qattr[0].val.clusterDim.z = 1;
        qcfg.attrs = qattr;
        qcfg.numAttrs = 1;
        int resident = 0;
        if (cudaOccupancyMaxActiveClusters(&resident, kernel, &qcfg) == cudaSuccess &&
            resident >= plp->tiles) {
          cluster = c;
          break;
        }
        cudaGetLastError();
      }
      cache[key] = cluster;
    }
  }
  if (cluster == 1) {
    const size_t need = kStatusBytes + counters_bytes(plp->tiles) +
                        static_cast<size_t>(plp->tiles) * plp->max_slots * plp->NU * kTileN * sizeof(float);
    if (workspace_bytes < need) {
      // The workspace was sized for another grid cap: whole tiles need no partial sums.
      if (plp->max_slots > 1) plan = make_plan(M, N, K, BITS, di.sms, max_ctas, false);
      if (plp->max_slots > 1) return DXB_ERR_WORKSPACE;
    }
  }
  const Plan& pl = *plp;
  if (cluster == 1)
    kernel = pick_kernel<BITS, HAS_ZERO>(multi, relaid, lean && pl.whole ? kModeWhole : kModeGeneral);

  const CUtensorMap* tq = cached_map(MapKey{qw, N, pl.rows, 0, BITS}, [&](CUtensorMap* m) {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(pl.rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N)};
    const uint32_t box[2] = {kTileN, static_cast<uint32_t>(pl.unit_rows)};
    return make_map(m, qw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  });
  const CUtensorMap* tx = cached_map(MapKey{x, ldx, (static_cast<long long>(M) << 32) | K, pl.NU, 16 + BITS},
                                     [&](CUtensorMap* m) {
    if (BITS == 4) {
      // X seen as [plane][token][k within the plane]: one box brings both k-slices of a unit.
      const uint64_t dims[3] = {static_cast<uint64_t>(K / 2), static_cast<uint64_t>(M), 2};
      const uint64_t strides[2] = {static_cast<uint64_t>(ldx) * 2, static_cast<uint64_t>(K / 2) * 2};
      const uint32_t box[3] = {64, static_cast<uint32_t>(pl.NU), 2};
      return make_map(m, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldx) * 2};
    const uint32_t box[2] = {64, static_cast<uint32_t>(pl.NU)};
    return make_map(m, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  });
  if (!tq || !tx) return DXB_ERR_TENSORMAP;

  WqParams p{};
  p.scales = static_cast<const __nv_bfloat16*>(scales);
  p.zeros = static_cast<const __nv_bfloat16*>(zeros);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  uint8_t* wsb = static_cast<uint8_t*>(workspace);
  p.status = reinterpret_cast<int*>(wsb);
  p.counters = reinterpret_cast<int*>(wsb + kStatusBytes);
  p.partials = reinterpret_cast<float*>(wsb + kStatusBytes + counters_bytes(pl.tiles));
  p.M = M; p.N = N; p.K = K; p.group = group;
  p.NU = pl.NU;
  p.units_per_tile = pl.units_per_tile;
  p.tiles = pl.tiles;
  p.tiles_n = pl.tiles_n;
  p.total_units = pl.total_units;
  p.half_k = BITS == 4 ? K / 2 : 0;
  p.stages = pl.stages;
  p.w_stages = pl.w_stages;
  p.x_stage_bytes = pl.x_stage_bytes;
  p.max_slots = pl.max_slots;
  p.nacc = pl.nacc;
  {
    const int gu = group / kUnitRows;
    int sh = -1;
    for (int b = 0; b < 20; ++b) if ((1 << b) == gu) sh = b;
    p.group_shift = sh;
  }
  p.trace = g_trace;
  {
    static const int dbg = [] { const char* e = getenv("DXB_DEBUG"); return e ? atoi(e) : 0; }();
    p.debug = dbg;
  }
  p.epilogue = opts.epilogue;
  p.tile_ranges = (cluster == 1 && pl.whole) ? 1 : 0;
  p.peer = opts.peer;
  p.cluster = cluster;
  p.recv_off = pl.recv_off;
  p.recv_alias = cluster > 1 ? pl.recv_alias : 0;
  p.rows_per = ((M > 128 ? 128 : M) + cluster - 1) / cluster;  // token rows of one block per CTA
  {
    const int what = cluster > 1 ? pl.units_per_tile : pl.tiles;
    const int parts = cluster > 1 ? cluster : pl.ctas;
    p.range_q = what / parts;
    p.range_r = what % parts;
  }
  p.rows_inv = (65536 + p.rows_per - 1) / p.rows_per;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster > 1 ? pl.tiles * cluster : pl.ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (cluster > 1) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = cluster;
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  if (pdl_enabled() && !opts.serialize) {
    // Let this launch begin while the previous kernel of the stream drains: the kernel
    // itself waits (griddepcontrol.wait) before touching anything that kernel may produce.
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  if (cudaLaunchKernelEx(&cfg, kernel, *tq, *tx, p) != cudaSuccess) {
    cudaGetLastError();
    return DXB_ERR_CUDA;
  }
  return cudaGetLastError() == cudaSuccess ? DXB_OK : DXB_ERR_CUDA;
}

template <int BITS>
static int launch_simt(const void* x, long long ldx, const void* qw, const void* scales,
                       const void* zeros, const void* bias, void* out, long long ldo, int M, int N,
                       int K, int group, const Opts& opts, cudaStream_t stream) {
  dim3 block(128), grid((N + 127) / 128, (M + 7) / 8);
  wq_gemm_simt<BITS><<<grid, block, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const uint8_t*>(qw),
      static_cast<const __nv_bfloat16*>(scales), static_cast<const __nv_bfloat16*>(zeros),
      static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(out), ldo, M, N, K, group,
      opts.relaid, opts.epilogue);
  return cudaGetLastError() == cudaSuccess ? DXB_OK : DXB_ERR_CUDA;
}

static int check_args(int bits, const void* x, long long ldx, const void* qw, const void* scales,
                      void* out, long long ldo, int M, int N, int K, int group) {
  if (bits != 4 && bits != 8) return DXB_ERR_BITS;
  if (!x || !qw || !scales || !out) return DXB_ERR_NULL;
  if (M < 0 || N <= 0 || K <= 0 || group <= 0) return DXB_ERR_SHAPE;
  if (K % group) return DXB_ERR_SHAPE;
  if (bits == 4 && (K % 2)) return DXB_ERR_SHAPE;
  if (ldx < K || ldo < N) return DXB_ERR_SHAPE;
  return DXB_OK;
}

static bool pointers_aligned(int bits, const void* x, long long ldx, const void* qweight, const void* scales,
                             const void* zeros, const void* bias, const void* out, long long ldo, int K) {
  return (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (ldx % 8 == 0) &&
         (reinterpret_cast<uintptr_t>(qweight) % 16 == 0) && (reinterpret_cast<uintptr_t>(scales) % 16 == 0) &&
         (zeros == nullptr || reinterpret_cast<uintptr_t>(zeros) % 16 == 0) &&
         (bias == nullptr || reinterpret_cast<uintptr_t>(bias) % 8 == 0) &&
         (reinterpret_cast<uintptr_t>(out) % 8 == 0) && (ldo % 4 == 0) && (bits != 4 || (K / 2) % 8 == 0);
}

// Checks dxb_gemm_opts against the problem and copies it.
static int read_opts(const dxb_gemm_opts* o, int bits, int M, int N, int K, Opts* out) {
  Opts r;
  if (o) {
    if (o->weight_layout != DXB_LAYOUT_DEXTER && o->weight_layout != DXB_LAYOUT_B200) return DXB_ERR_UNSUPPORTED;
    if (o->weight_layout == DXB_LAYOUT_B200 && (bits != 4 || (K / 2) % 2 || N % 4)) return DXB_ERR_UNSUPPORTED;
    if (o->epilogue != DXB_EPILOGUE_NONE && o->epilogue != DXB_EPILOGUE_GELU_TANH) return DXB_ERR_UNSUPPORTED;
    r.relaid = o->weight_layout == DXB_LAYOUT_B200;
    r.epilogue = o->epilogue;
    r.max_ctas = o->max_ctas;
    r.serialize = o->serialize;
    if (o->peer_world > 1) {
      if (o->peer_world > kPeerMaxRanks || o->peer_rank < 0 || o->peer_rank >= o->peer_world) return DXB_ERR_SHAPE;
      if (!o->peer_regions) return DXB_ERR_NULL;
      // one token block, whole 4-column groups, a counter per tile, room for the partial output
      if (M > 128 || N % 4 || (N + kTileN - 1) / kTileN > kFusedMaxTiles) return DXB_ERR_UNSUPPORTED;
      if (o->peer_capacity_elems < static_cast<int64_t>(M) * N) return DXB_ERR_SHAPE;
      for (int i = 0; i < o->peer_world; ++i) {
        if (!o->peer_regions[i] || reinterpret_cast<uintptr_t>(o->peer_regions[i]) % 16) return DXB_ERR_NULL;
        r.peer.region[i] = static_cast<unsigned char*>(o->peer_regions[i]);
      }
      r.peer.capacity = o->peer_capacity_elems;
      r.peer.rank = o->peer_rank;
      r.peer.world = o->peer_world;
      r.peer.wait_tries = wait_tries();
    }
  }
  *out = r;
  return DXB_OK;
}

static int gemm_dispatch(int bits, const void* x, int64_t ldx, const void* qweight, const void* scales,
                         const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
                         int group_size, void* workspace, size_t workspace_bytes, const Opts& opts,
                         cudaStream_t stream) {
  const int max_ctas = opts.max_ctas;
  const bool aligned = pointers_aligned(bits, x, ldx, qweight, scales, zeros, bias, out, ldo, K);
  auto launch = [&](const char* xc, char* oc, int mc) -> int {
    if (bits == 4)
      return zeros ? launch_tc<4, true>(xc, ldx, qweight, scales, zeros, bias, oc, ldo, mc, N, K,
                                        group_size, workspace, workspace_bytes, opts, stream)
                   : launch_tc<4, false>(xc, ldx, qweight, scales, zeros, bias, oc, ldo, mc, N, K,
                                         group_size, workspace, workspace_bytes, opts, stream);
    return zeros ? launch_tc<8, true>(xc, ldx, qweight, scales, zeros, bias, oc, ldo, mc, N, K,
                                      group_size, workspace, workspace_bytes, opts, stream)
                 : launch_tc<8, false>(xc, ldx, qweight, scales, zeros, bias, oc, ldo, mc, N, K,
                                       group_size, workspace, workspace_bytes, opts, stream);
  };
  // The sum over ranks lives in the tensor-core kernel's epilogue only.
  if (opts.peer.world > 1 && !(aligned && gemm_tc_supported(M, N, K, group_size, bits)))
    return DXB_ERR_UNSUPPORTED;
  // More than 128 tokens: one launch over all token blocks when the workspace holds the
  // partial sums of that plan (dxb_workspace_bytes asks for it); a smaller workspace still
  // works, block by block.
  if (M > 128 && aligned && gemm_tc_supported(M, N, K, group_size, bits) &&
      workspace_bytes >= plan_workspace_bytes(M, N, K, bits, max_ctas))
    return launch(static_cast<const char*>(x), static_cast<char*>(out), M);
  // Token blocks of at most 128 rows per launch (the UMMA N of one accumulator); 96 when the
  // weight has so few tiles that the launch splits them over clusters, whose receive buffers
  // only fit next to the activation ring up to 96 tokens.
  int chunk = M <= 128 ? M : 128;
  if (M > 128 && ((N + kTileN - 1) / kTileN) * 2 <= device_info().sms) chunk = 96;
  for (int m0 = 0; m0 < M; m0 += chunk) {
    const int mc = (M - m0) < chunk ? (M - m0) : chunk;
    const char* xc = static_cast<const char*>(x) + static_cast<long long>(m0) * ldx * 2;
    char* oc = static_cast<char*>(out) + static_cast<long long>(m0) * ldo * 2;
    int rc;
    if (aligned && gemm_tc_supported(mc, N, K, group_size, bits)) {
      rc = launch(xc, oc, mc);
    } else {
      rc = bits == 4 ? launch_simt<4>(xc, ldx, qweight, scales, zeros, bias, oc, ldo, mc, N, K,
                                      group_size, opts, stream)
                     : launch_simt<8>(xc, ldx, qweight, scales, zeros, bias, oc, ldo, mc, N, K,
                                      group_size, opts, stream);
    }
    if (rc != DXB_OK) return rc;
  }
  return DXB_OK;
}

}  // namespace dx

// =================================================================== C ABI ==
extern "C" {

#ifdef DXB_TRACE
void dxb_debug_set_trace(void* ptr) { dx::g_trace = static_cast<long long*>(ptr); }
#endif

int dxb_wq_gemm_ex(int bits, const void* x, int64_t ldx, const void* qweight, const void* scales,
                   const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
                   int group_size, void* workspace, size_t workspace_bytes, const dxb_gemm_opts* opts,
                   void* cuda_stream) {
  using namespace dx;
  int rc = check_args(bits, x, ldx, qweight, scales, out, ldo, M, N, K, group_size);
  if (rc != DXB_OK) return rc;
  Opts o;
  rc = read_opts(opts, bits, M, N, K, &o);
  if (rc != DXB_OK) return rc;
  if (M == 0) return DXB_OK;
  return gemm_dispatch(bits, x, ldx, qweight, scales, zeros, bias, out, ldo, M, N, K, group_size, workspace,
                       workspace_bytes, o, static_cast<cudaStream_t>(cuda_stream));
}

int dxb_wq_gemm(int bits, const void* x, int64_t ldx, const void* qweight, const void* scales,
                const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
                int group_size, void* workspace, size_t workspace_bytes, int max_ctas,
                void* cuda_stream) {
  dxb_gemm_opts o = {};
  o.max_ctas = max_ctas;
  return dxb_wq_gemm_ex(bits, x, ldx, qweight, scales, zeros, bias, out, ldo, M, N, K, group_size, workspace,
                        workspace_bytes, &o, cuda_stream);
}

// ---------------------------------------------------------------------------
// Scratch that lives inside the library image, for callers that must not
// allocate device memory (see dxb_wq_gemm_static in the header).  Zero at load
// time; every GPU that loads the library keeps these 24 MiB until the process
// exits.  In host code the symbol below is only a stand-in: its device address
// has to be asked for with cudaGetSymbolAddress, per device.
constexpr size_t kStaticScratchBytes = static_cast<size_t>(24) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace dx {
constexpr int kMaxDevices = 64;
// Device address of g_static_scratch on the CURRENT device, looked up once per device.
static int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* addr[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return DXB_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();  // clear the sticky-less error so later calls start clean
      return DXB_ERR_CUDA;
    }
    addr[dev] = p;
  }
  *out = addr[dev];
  return DXB_OK;
}
}  // namespace dx

int dxb_wq_gemm_static(int bits, const void* x, int64_t ldx, const void* qweight,
                       const void* scales, const void* zeros, const void* bias, void* out,
                       int64_t ldo, int M, int N, int K, int group_size, void* cuda_stream) {
  using namespace dx;
  int rc = check_args(bits, x, ldx, qweight, scales, out, ldo, M, N, K, group_size);
  if (rc != DXB_OK) return rc;
  if (M == 0) return DXB_OK;
  // What one launch of at most 128 tokens needs; with more tokens dxb_wq_gemm takes the
  // one-launch plan when the array holds it and goes block by block otherwise.  Shapes that
  // run on the plain CUDA-core kernel use no scratch at all.
  const int mc = M <= 128 ? M : 128;
  if (pointers_aligned(bits, x, ldx, qweight, scales, zeros, bias, out, ldo, K) &&
      gemm_tc_supported(mc, N, K, group_size, bits) &&
      (plan_workspace_bytes(mc, N, K, bits, 0) > kStaticScratchBytes ||
       (M > 128 && plan_workspace_bytes(96, N, K, bits, 0) > kStaticScratchBytes)))
    return DXB_ERR_SCRATCH_LIMIT;
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != DXB_OK) return rc;
  // The array keeps whatever the previous call left.  Partial sums are always written
  // before they are read, but the tile counters must start at zero.  The status word in
  // front of them is left alone: a timeout reported by an earlier call stays readable
  // (dxb_read_status(NULL, stream)) until it has been read.
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (cudaMemsetAsync(static_cast<unsigned char*>(scratch) + kStatusBytes, 0, counters_bytes(0), stream) !=
      cudaSuccess)
    return DXB_ERR_CUDA;
  return dxb_wq_gemm(bits, x, ldx, qweight, scales, zeros, bias, out, ldo, M, N, K, group_size,
                     scratch, kStaticScratchBytes, 0, cuda_stream);
}

int dxb_w4a16(const void* x, int64_t ldx, const void* qweight, const void* scales,
              const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
              int group_size, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  return dxb_wq_gemm(4, x, ldx, qweight, scales, zeros, bias, out, ldo, M, N, K, group_size,
                     workspace, workspace_bytes, 0, cuda_stream);
}

int dxb_w8a16(const void* x, int64_t ldx, const void* qweight, const void* scales,
              const void* zeros, const void* bias, void* out, int64_t ldo, int M, int N, int K,
              int group_size, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  return dxb_wq_gemm(8, x, ldx, qweight, scales, zeros, bias, out, ldo, M, N, K, group_size,
                     workspace, workspace_bytes, 0, cuda_stream);
}

size_t dxb_workspace_bytes_ex(int M, int N, int K, int bits, int max_ctas) {
  using namespace dx;
  if (M <= 0 || N <= 0 || K <= 0 || (bits != 4 && bits != 8)) return kStatusBytes;
  const int rows = bits == 4 ? K / 2 : K;
  if (rows < (bits == 4 ? 64 : 128)) return kStatusBytes;
  // Up to 128 tokens: that launch.  More: the larger of the one-launch plan over all token
  // blocks and the plan of a single block (used when the caller's workspace is smaller).
  size_t one_block = plan_workspace_bytes(M <= 128 ? M : 128, N, K, bits, max_ctas);
  if (M <= 128) return one_block;
  // block by block, few-tile weights go in blocks of 96 tokens (see dxb_wq_gemm)
  const size_t block96 = plan_workspace_bytes(96, N, K, bits, max_ctas);
  if (block96 > one_block) one_block = block96;
  if (static_cast<long long>((N + kTileN - 1) / kTileN) * ((M + 127) / 128) > kMaxTiles)
    return one_block;
  const size_t all_blocks = plan_workspace_bytes(M, N, K, bits, max_ctas);
  return all_blocks > one_block ? all_blocks : one_block;
}

size_t dxb_workspace_bytes(int M, int N, int K, int bits) { return dxb_workspace_bytes_ex(M, N, K, bits, 0); }

int dxb_relayout_w4(const void* qweight, void* out, int K, int N, int inverse, void* cuda_stream) {
  using namespace dx;
  if (!qweight || !out) return DXB_ERR_NULL;
  if (K <= 0 || N <= 0 || K % 4 || N % 4) return DXB_ERR_SHAPE;  // whole row pairs, whole 32-bit words
  if (reinterpret_cast<uintptr_t>(qweight) % 4 || reinterpret_cast<uintptr_t>(out) % 4) return DXB_ERR_UNSUPPORTED;
  const long long row_pairs = K / 4;
  const int n4 = N / 4;
  const long long total = row_pairs * n4;
  const int block = 256;
  wq_relayout_w4_kernel<<<static_cast<unsigned>((total + block - 1) / block), block, 0,
                          static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint32_t*>(qweight), static_cast<uint32_t*>(out), row_pairs, n4, inverse ? 1 : 0);
  return cudaGetLastError() == cudaSuccess ? DXB_OK : DXB_ERR_CUDA;
}

size_t dxb_fused_reduce_bytes(int world, int64_t capacity_elems) {
  if (world < 1 || world > dx::kPeerMaxRanks || capacity_elems <= 0) return 0;
  const size_t cap = (static_cast<size_t>(capacity_elems) + 7) / 8 * 8;
  return dx::kFusedHeaderBytes + 2 * static_cast<size_t>(world) * cap * 2;
}

void dxb_set_wait_limit_ms(int ms) {
  const long long tries = static_cast<long long>(ms < 1 ? 1 : ms) * 4000;
  dx::g_wait_tries.store(static_cast<unsigned>(tries > 4000000000ll ? 4000000000ll : tries));
}

int dxb_dequantize_ex(const void* qweight, const void* scales, const void* zeros, void* w_out, int N,
                      int K, int group_size, int bits, int weight_layout, void* cuda_stream) {
  using namespace dx;
  if (bits != 4 && bits != 8) return DXB_ERR_BITS;
  if (!qweight || !scales || !w_out) return DXB_ERR_NULL;
  if (N <= 0 || K <= 0 || group_size <= 0 || K % group_size || (bits == 4 && K % 2))
    return DXB_ERR_SHAPE;
  if (weight_layout != DXB_LAYOUT_DEXTER && (weight_layout != DXB_LAYOUT_B200 || bits != 4 || K % 4 || N % 4))
    return DXB_ERR_UNSUPPORTED;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const long long total = static_cast<long long>(K) * N;
  const int block = 256;
  const unsigned grid = static_cast<unsigned>((total + block - 1) / block);
  if (bits == 4)
    wq_dequant_kernel<4><<<grid, block, 0, stream>>>(
        static_cast<const uint8_t*>(qweight), static_cast<const __nv_bfloat16*>(scales),
        static_cast<const __nv_bfloat16*>(zeros), static_cast<__nv_bfloat16*>(w_out), N, K, group_size,
        weight_layout == DXB_LAYOUT_B200);
  else
    wq_dequant_kernel<8><<<grid, block, 0, stream>>>(
        static_cast<const uint8_t*>(qweight), static_cast<const __nv_bfloat16*>(scales),
        static_cast<const __nv_bfloat16*>(zeros), static_cast<__nv_bfloat16*>(w_out), N, K, group_size, 0);
  return cudaGetLastError() == cudaSuccess ? DXB_OK : DXB_ERR_CUDA;
}

int dxb_dequantize(const void* qweight, const void* scales, const void* zeros, void* w_out, int N,
                   int K, int group_size, int bits, void* cuda_stream) {
  return dxb_dequantize_ex(qweight, scales, zeros, w_out, N, K, group_size, bits, DXB_LAYOUT_DEXTER, cuda_stream);
}

int dxb_uses_tensor_cores(int M, int N, int K, int group_size, int bits) {
  const int mc = M <= 128 ? M : 128;
  return dx::gemm_tc_supported(mc, N, K, group_size, bits) ? 1 : 0;
}

int dxb_read_status(void* workspace, void* cuda_stream) {
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const bool builtin = workspace == nullptr;  // the scratch of dxb_wq_gemm_static
  if (builtin && dx::static_scratch_address(&workspace) != DXB_OK) return DXB_ERR_CUDA;
  int code = 0;
  if (cudaMemcpyAsync(&code, workspace, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
    return DXB_ERR_CUDA;
  // The built-in scratch has no owner who could clear its status word: reading it does.
  if (builtin && cudaMemsetAsync(workspace, 0, sizeof(int), stream) != cudaSuccess) return DXB_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return DXB_ERR_CUDA;
  return code;
}

const char* dxb_strerror(int code) {
  switch (code) {
    case DXB_OK: return "ok";
    case DXB_ERR_BITS: return "bits must be 4 or 8";
    case DXB_ERR_NULL: return "null pointer argument";
    case DXB_ERR_SHAPE: return "inconsistent shape, stride or group size";
    case DXB_ERR_UNSUPPORTED: return "shape or option not supported by this build";
    case DXB_ERR_WORKSPACE: return "workspace missing or too small (see dxb_workspace_bytes)";
    case DXB_ERR_TENSORMAP: return "could not encode a TMA tensor map";
    case DXB_ERR_CUDA: return "CUDA launch or runtime error";
    case DXB_ERR_KERNEL_TIMEOUT: return "a bounded wait inside the kernel ran out";
    case DXB_ERR_SCRATCH_LIMIT:
      return "problem needs more scratch than the 24 MiB built into the library "
             "(use dxb_wq_gemm with a caller-provided workspace)";
    default: return "unknown error";
  }
}

}  // extern "C"
