// A list of weight-only quantised GEMMs (the linears of one layer) in one launch.
//
// One persistent CTA per SM runs the same warp-specialised pipeline as wq_gemm_tc
// (TMA producers -> dequant teams writing TMEM -> one MMA issuer -> epilogue warps),
// but every role walks through ALL items of the list: item i+1's packed weights are
// loaded and converted while item i's last MMAs and epilogue drain, so the start-up
// and drain that dominate a single launch at <= 128 tokens are paid once per list.
//
// Work split: the grid is a set of thread-block clusters of C CTAs.  The tiles (128
// weight columns) of all items are dealt round-robin to the clusters; the C CTAs of a
// cluster split the K range of each of their tiles evenly and add their partial sums
// through distributed shared memory: CTA r of the cluster finishes token rows
// [r*rows_per, (r+1)*rows_per); every CTA stores each owner's rows of its fp32 partial
// tile straight into the owner's receive buffer and arrives (release, cluster scope)
// on a barrier in the owner's shared memory; the owner waits on that barrier, adds
// the C buffers in rank order (deterministic), adds the bias and writes bf16.  A second
// barrier, on which the owners arrive remotely, tells every CTA when the receive
// buffers it wrote may be overwritten with the next tile.  No partial sum touches
// global memory, and all waits on other CTAs stay inside one cluster, whose CTAs the
// hardware schedules together.
//
// Hand-over between items: the epilogue counts finished (tile, owner) shares per item
// (done[item]) for every item that a later one depends on; the activation producer of
// the dependent item waits (bounded) until that count is complete, then orders its TMA
// reads after that observation with a proxy fence.  This is the one wait that crosses
// clusters, which is why the grid is sized to be resident at once.
#include "wq_common.cuh"

namespace dx {
#ifdef DXB_TRACE
#define CH_TRACE(role, i) do { if (P.trace && (i) < 64) P.trace[(static_cast<long long>(blockIdx.x) * 8 + (role)) * 64 + (i)] = clock64() - t_start; } while (0)
#else
#define CH_TRACE(role, i) do { } while (0)
#endif

constexpr int kMaxChain = DXB_CHAIN_MAX;
constexpr int kAccStride = 128;  // TMEM columns between the two accumulators
// Four more barriers behind the pipeline's own: one pair per receive buffer.
constexpr int kBarRecvFull = kNumBars;      // [2] every CTA's rows of this tile have arrived here
constexpr int kBarPeerFree = kNumBars + 2;  // [2] every owner has read what this CTA sent
constexpr int kChainBars = kNumBars + 4;

struct ChainItem {
  const __nv_bfloat16* scales;
  const __nv_bfloat16* zeros;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  long long ldo;
  int M, N, NU;
  int U;            // units per tile
  int tiles;
  int half_units;   // int4: units between the low- and the high-nibble plane of scales
  int group_shift;  // log2(group / 64) or -1
  int group_units;  // group / 64
  int x_bytes;      // bytes one unit of activations brings
  int dep;          // item whose output is this item's activations, or -1
  int rot;          // cluster that takes tile 0 of this item
  int need_done;    // a later item depends on this one: count finished shares
  int rows_per;     // token rows each CTA of a cluster finishes: ceil(M / C)
  int rows_inv;     // ceil(65536 / rows_per): row / rows_per == (row * rows_inv) >> 16
};

struct ChainParams {
  CUtensorMap tm_q[kMaxChain];
  CUtensorMap tm_x[kMaxChain];
  ChainItem item[kMaxChain];
  int* status;
  int* done;  // [kMaxChain] finished (tile, owner) shares per item
  int* exits; // CTAs that have finished; the last one clears `done` for the next launch
  int n;
  int w_stages;
  int x_stage_bytes;  // ring stride: the largest x_bytes of the list
  int recv_off;       // byte offset of the receive buffers in shared memory
  int recv_bytes;     // bytes of one receive buffer (C x rows_per x 128 fp32)
  int recv_bufs;      // 2 when two receive buffers fit next to the rings, else 1
  int cluster;        // C
  int pad_;
  long long* trace;   // only used when built with -DDXB_TRACE
};

// One owner's share of a tile: rows [m_lo, m_hi) of the CC receive buffers (one per CTA of
// the cluster, `src_stride` bytes apart) added in rank order, bias added the way the
// reference does (round the matmul to bf16, then add in bf16), written as bf16.
// 128 threads: thread `etid` takes columns 4*(etid % 32).. and every fourth row.
template <int CC>
__device__ __forceinline__ void chain_sum_rows(uint32_t rbase, uint32_t src_stride, int m_lo, int m_hi,
                                               int etid, bool has_bias, const float (&bias4)[4],
                                               __nv_bfloat16* out_col, long long ldo) {
  const uint32_t col_off = static_cast<uint32_t>((etid & 31) * 16);
  uint32_t a0 = rbase + static_cast<uint32_t>(etid >> 5) * (kTileN * 4u) + col_off;
  __nv_bfloat16* dst = out_col + static_cast<long long>(m_lo + (etid >> 5)) * ldo;
  const long long dst_step = ldo * (kEpilogueThreads / 32);
  for (int m = m_lo + (etid >> 5); m < m_hi; m += kEpilogueThreads / 32) {
    float4 v[CC];
#pragma unroll
    for (int rr = 0; rr < CC; ++rr) v[rr] = ld_smem_f4(a0 + rr * src_stride);
    float4 acc = v[0];
#pragma unroll
    for (int rr = 1; rr < CC; ++rr) {  // rank order: the sum does not depend on timing
      acc.x += v[rr].x; acc.y += v[rr].y; acc.z += v[rr].z; acc.w += v[rr].w;
    }
    uint2 pk;
    if (has_bias) {
      const uint32_t r01 = cvt_bf16x2(acc.y, acc.x), r23 = cvt_bf16x2(acc.w, acc.z);
      pk.x = cvt_bf16x2(bf16hi_f32(r01) + bias4[1], bf16lo_f32(r01) + bias4[0]);
      pk.y = cvt_bf16x2(bf16hi_f32(r23) + bias4[3], bf16lo_f32(r23) + bias4[2]);
    } else {
      pk.x = cvt_bf16x2(acc.y, acc.x);
      pk.y = cvt_bf16x2(acc.w, acc.z);
    }
    *reinterpret_cast<uint2*>(dst) = pk;
    a0 += (kEpilogueThreads / 32) * (kTileN * 4u);
    dst += dst_step;
  }
}

template <int BITS, bool HAS_ZERO>
__global__ void __launch_bounds__(kThreads, 1)
wq_chain_tc(const __grid_constant__ ChainParams P) {
  constexpr int PLANES = BITS == 4 ? 2 : 1;
  constexpr int A_STAGE_COLS = PLANES * 32;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[kChainBars];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  // Where the epilogue sends accumulator row m of the current item: cluster address of that
  // row (column 0, receive buffer 0) in its owner's shared memory, or ~0 for rows >= M.
  // Entry [16*i + 4*c + rep] is row 16*i + 4*rep + c: the four rows one thread holds after
  // one accumulator load sit side by side.
  __shared__ __align__(16) uint32_t dst_tab[128];
#ifdef DXB_TRACE
  __shared__ long long t_start;
  if (threadIdx.x == 0) t_start = clock64();
  __syncthreads();
#endif

  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t w_ring = smem0;
  const uint32_t x_ring = smem0 + P.w_stages * kWStage;
  const uint32_t recv0 = smem0 + static_cast<uint32_t>(P.recv_off);
  const uint32_t bar0 = smem_u32(bars);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int SW = P.w_stages;
  const int C = P.cluster;
  const int NC = static_cast<int>(gridDim.x) / C;   // clusters
  const int cid = static_cast<int>(blockIdx.x) / C; // this cluster
  const int r = static_cast<int>(blockIdx.x) % C;   // rank in the cluster (1-D clusters)
  const int NI = P.n;

  if (warp == 3) {
    for (int i = lane; i < kChainBars; i += 32)
      mbar_init(bar0 + 8 * i, i < kNumBars ? bar_count(i) : static_cast<uint32_t>(4 * C));
    if (lane == 0) abort_flag = 0;
    mbar_init_fence();
  } else if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&P.tm_q[0]);
  } else if (warp == 2 && lane == 0) {
    tma_prefetch_desc(&P.tm_x[0]);
  } else if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Peers arrive on this CTA's barriers: nobody may start before all are initialised.
  cluster_sync_all();
  const uint32_t tmem0 = tmem_base_s;
  volatile int* abortp = &abort_flag;

  // Tiles of item j that this cluster takes: first_tile(j), + NC, + 2 NC, ...; this CTA's
  // K units of every such tile: [kb, ke).
  auto first_tile = [&](int j) {
    int t = cid - P.item[j].rot;
    return t < 0 ? t + NC : t;
  };
  auto unit_range = [&](int j, int& kb, int& ke) {
    const int U = P.item[j].U;
    kb = r * U / C;
    ke = (r + 1) * U / C;
  };

  // All roles number the units this CTA processes 0, 1, 2, ... across the whole list.
  // Ring stages, TMEM slots and barrier phases follow that running number, so they carry
  // over from tile to tile and from item to item.
  if (warp == 0 || warp == 3) {
    // ============================================ TMA producer: packed weights
    // Warps 0 and 3 take the even and the odd running numbers.
    const int pi = warp == 0 ? 0 : 1;
    int s = pi, n = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int j = 0; j < NI && ok; ++j) {
      int kb, ke;
      unit_range(j, kb, ke);
      const int tiles = P.item[j].tiles;
      if (j + 1 < NI && lane == 0) tma_prefetch_desc(&P.tm_q[j + 1]);
      for (int tile = first_tile(j); tile < tiles && ok; tile += NC) {
        int ku = kb + ((pi - n) & 1);
        n += ke - kb;
        for (; ku < ke; ku += 2) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar0 + 8 * (kBarEmptyW + s), ph ^ 1u, abortp));
          if (!ok) break;
          if (elect_one()) {
            const uint32_t fw = bar0 + 8 * (kBarFullW + s);
            mbar_expect_tx(fw, kQBytes);
            tma_load_2d(w_ring + s * kWStage, &P.tm_q[j], fw, tile * kTileN, ku * kUnitRows);
          }
          __syncwarp();
          s += 2;
          if (s >= SW) { s -= SW; ph ^= 1u; }
        }
      }
    }
    if (!ok && lane == 0) {
      // Leaving early: let the copies already issued land before the CTA exits.
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000) {}
    }
    __syncwarp();
  } else if (warp == 2) {
    // ============================================== TMA producer: activations
    pdl_wait();
    int t = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int j = 0; j < NI && ok; ++j) {
      int kb, ke;
      unit_range(j, kb, ke);
      const int tiles = P.item[j].tiles;
      int tile = first_tile(j);
      if (tile >= tiles || kb >= ke) continue;
      const int dep = P.item[j].dep;
      if (dep >= 0) {
        // The activations are item `dep`'s output: wait until all its shares are written.
        bool fine = true;
        if (lane == 0) fine = wait_flag_ge(P.done + dep, P.item[dep].tiles * C, abortp);
        ok = __shfl_sync(0xffffffffu, fine ? 1 : 0, 0) != 0;
        if (!ok) break;
        fence_proxy_async_all();  // the TMA reads below come after that observation
      }
      if (j + 1 < NI && lane == 0) tma_prefetch_desc(&P.tm_x[j + 1]);
      const uint32_t x_bytes = static_cast<uint32_t>(P.item[j].x_bytes);
      for (; tile < tiles && ok; tile += NC) {
        for (int ku = kb; ku < ke; ++ku) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar0 + 8 * (kBarFree + t), ph ^ 1u, abortp));
          if (!ok) break;
          if (elect_one()) {
            const uint32_t rb = bar0 + 8 * (kBarReady + t);
            mbar_expect_tx(rb, x_bytes);
            if (BITS == 4)
              tma_load_3d(x_ring + t * P.x_stage_bytes, &P.tm_x[j], rb, ku * kUnitRows, 0, 0);
            else
              tma_load_2d(x_ring + t * P.x_stage_bytes, &P.tm_x[j], rb, ku * kUnitRows, 0);
          }
          __syncwarp();
          if (++t == kAStages) { t = 0; ph ^= 1u; }
        }
      }
    }
    if (!ok && lane == 0) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000) {}
    }
    __syncwarp();
  } else if (warp == 1) {
    // ======================================================= MMA issuer ====
    const uint64_t xdesc0 = smem_desc_kmajor_sw128(x_ring);
    const uint32_t x_stage16 = static_cast<uint32_t>(P.x_stage_bytes) >> 4;
    int t = 0, b = 0;
    uint32_t ph = 0, accph = 0;
    uint64_t xd = xdesc0;
    uint32_t a_tmem = tmem0 + kACol0;
    bool ok = true;
    const bool leader = elect_one();  // the one lane that issues; fixed for the whole loop
    int mcount = 0;
    (void)mcount;
    for (int j = 0; j < NI && ok; ++j) {
      int kb, ke;
      unit_range(j, kb, ke);
      const int tiles = P.item[j].tiles;
      const int nun = ke - kb;
      if (nun <= 0) continue;
      const uint32_t idesc = idesc_bf16_f32(kTileN, P.item[j].NU);
      const uint32_t plane16 = static_cast<uint32_t>(P.item[j].NU * 128) >> 4;
      for (int tile = first_tile(j); tile < tiles && ok; tile += NC) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar0 + 8 * (kBarAccEmpty + b), accph ^ 1u, abortp));
        if (!ok) break;
        const uint32_t d_tmem = tmem0 + b * kAccStride;
        uint32_t accumulate = 0;
        for (int i = 0; i < nun; ++i) {
          if (!mbar_wait(bar0 + 8 * (kBarReady + t), ph, abortp)) { ok = false; break; }
          tc_fence_after();
          if (leader) {
            mma_ts(d_tmem, a_tmem, xd, idesc, accumulate);
#pragma unroll
            for (int kk = 1; kk < 4; ++kk) mma_ts(d_tmem, a_tmem + kk * 8, xd + kk * 2, idesc, 1u);
            if (PLANES == 2) {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                mma_ts(d_tmem, a_tmem + 32 + kk * 8, xd + plane16 + kk * 2, idesc, 1u);
            }
            tc_commit(bar0 + 8 * (kBarFree + t));
          }
          accumulate = 1;
          xd += x_stage16;
          a_tmem += A_STAGE_COLS;
          if (++t == kAStages) { t = 0; ph ^= 1u; xd = xdesc0; a_tmem = tmem0 + kACol0; }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (leader) tc_commit(bar0 + 8 * (kBarAccFull + b));
        if (lane == 0) CH_TRACE(7, mcount);
        ++mcount;
        if (++b == 2) { b = 0; accph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // ========================================================= epilogue ====
    // Accumulator lane 32q + 8b + g holds weight column 32q + 4g + b, so the 16x128b
    // load shape hands thread (g, c) the four consecutive columns 4g..4g+3 of token
    // 4*rep + c.
    pdl_wait();
    const int q = warp & 3;
    const int etid = (warp - 4) * 32 + lane;
    const int c = lane & 3;
    const int g = lane >> 2;
    const int n_local = 32 * q + 4 * g;
    const int NB = P.recv_bufs;
    // Lane l < C signals CTA l of the cluster.
    const uint32_t remote_bars = dsmem_addr(bar0, lane < C ? lane : 0);
    int b = 0;
    uint32_t accph = 0;
    int kbuf = 0;       // receive buffer of the next tile
    uint32_t bufph = 0; // its phase (flips each time the buffers wrap)
    bool ok = true;
    // A tile whose rows have been sent but whose own share is not summed yet.  With two
    // receive buffers the sum of tile k is put off until tile k+1 has been sent (when its
    // accumulator is already waiting), so the barrier round trips of one tile hide behind
    // the copies of the next; with one buffer, or when no accumulator is ready, it is
    // summed first.  Either order is safe: sending needs the owners to have read the tile
    // that last used the buffer, summing needs every CTA to have sent this tile, and every
    // CTA sends tile k before it does anything for tile k+1.
    int pj = -1, ptile = 0, pbuf = 0;
    uint32_t pph = 0;
    int tcount = 0, fcount = 0;  // tiles sent / finished (trace index)
    (void)tcount; (void)fcount;
    auto finish_pending = [&]() -> bool {
      const ChainItem& it = P.item[pj];
      const int M = it.M, N = it.N;
      const int rows_per = it.rows_per;
      const int m_lo = r * rows_per;
      const int m_hi = (m_lo + rows_per) < M ? (m_lo + rows_per) : M;
      const uint32_t src_stride = static_cast<uint32_t>(rows_per * kTileN) * 4u;
      const int col4 = (etid & 31) * 4;
      const int nn = ptile * kTileN + col4;
      const bool has_bias = it.bias != nullptr;
      float bias4[4] = {0.f, 0.f, 0.f, 0.f};
      if (has_bias && nn < N) {  // fetched before the wait below
        const uint2 bb = __ldg(reinterpret_cast<const uint2*>(it.bias + nn));
        bias4[0] = bf16lo_f32(bb.x); bias4[1] = bf16hi_f32(bb.x);
        bias4[2] = bf16lo_f32(bb.y); bias4[3] = bf16hi_f32(bb.y);
      }
      const uint32_t rbase = recv0 + static_cast<uint32_t>(pbuf * P.recv_bytes);
      if (etid == 0) CH_TRACE(4, fcount);
      if (!mbar_wait_cluster(bar0 + 8 * (kBarRecvFull + pbuf), pph, abortp)) return false;
      if (etid == 0) CH_TRACE(5, fcount);
      if (nn < N) {
        __nv_bfloat16* out_col = it.out + nn;
        if (C == 2)
          chain_sum_rows<2>(rbase, src_stride, m_lo, m_hi, etid, has_bias, bias4, out_col, it.ldo);
        else if (C == 4)
          chain_sum_rows<4>(rbase, src_stride, m_lo, m_hi, etid, has_bias, bias4, out_col, it.ldo);
        else
          chain_sum_rows<8>(rbase, src_stride, m_lo, m_hi, etid, has_bias, bias4, out_col, it.ldo);
      }
      __syncwarp();
      if (lane < C) mbar_arrive_remote(remote_bars + 8 * (kBarPeerFree + pbuf));  // this warp has read its part
      if (it.need_done) {
        fence_proxy_async_all();
        __threadfence();
        named_bar_sync(1, kEpilogueThreads);
        if (etid == 0) atomicAdd(P.done + pj, 1);
      }
      if (etid == 0) CH_TRACE(6, fcount);
      ++fcount;
      pj = -1;
      return true;
    };
    for (int j = 0; j < NI && ok; ++j) {
      int kb, ke;
      unit_range(j, kb, ke);
      if (kb >= ke) continue;
      const ChainItem& it = P.item[j];
      const int NU = it.NU;
      if (first_tile(j) >= it.tiles) continue;
      {
        // All four warps have sent the previous item's last tile before the table changes.
        named_bar_sync(2, kEpilogueThreads);
        const int m = (etid & ~15) + 4 * (etid & 3) + ((etid >> 2) & 3);
        uint32_t a = 0xFFFFFFFFu;
        if (m < it.M) {
          const int owner = (m * it.rows_inv) >> 16;
          const int row = r * it.rows_per + (m - owner * it.rows_per);
          a = dsmem_addr(recv0 + static_cast<uint32_t>(row * kTileN) * 4u, owner);
        }
        dst_tab[etid] = a;
        named_bar_sync(2, kEpilogueThreads);
      }
      const uint32_t tab = smem_u32(dst_tab) + static_cast<uint32_t>(c) * 16u;
      for (int tile = first_tile(j); tile < it.tiles && ok; tile += NC) {
        if (pj >= 0) {
          // Sum the waiting tile first unless the next accumulator is ready and its rows
          // can go to the other buffer (one lane decides for the warp).
          int later = 0;
          if (NB == 2 && lane == 0) later = mbar_try_wait(bar0 + 8 * (kBarAccFull + b), accph) ? 1 : 0;
          later = __shfl_sync(0xffffffffu, later, 0);
          if (!later) {
            ok = finish_pending();
            if (!ok) break;
          }
        }
        if (etid == 0) CH_TRACE(0, tcount);
        ok = mbar_wait(bar0 + 8 * (kBarAccFull + b), accph, abortp);
        if (!ok) break;
        tc_fence_after();
        if (etid == 0) CH_TRACE(1, tcount);
        // The owners must have read what this CTA last sent into this buffer.
        ok = mbar_wait_cluster(bar0 + 8 * (kBarPeerFree + kbuf), bufph ^ 1u, abortp);
        if (!ok) break;
        if (etid == 0) CH_TRACE(2, tcount);
        const uint32_t d_tmem = tmem_addr(tmem0 + b * kAccStride, 32 * q, 0);
        const uint32_t col_off = static_cast<uint32_t>(kbuf * P.recv_bytes + n_local * 4);
        for (int c0 = 0; c0 < NU; c0 += 16) {
          uint32_t ra[8], rb[8];
          tmem_ld_16x128b_x4(d_tmem + c0, ra);
          tmem_ld_16x128b_x4(d_tmem + (16u << 16) + c0, rb);
          const uint4 dst4 = lds128(tab + static_cast<uint32_t>(c0) * 4u);
          const uint32_t dst[4] = {dst4.x, dst4.y, dst4.z, dst4.w};
          tc_wait_ld();
#pragma unroll
          for (int rep = 0; rep < 4; ++rep) {
            if (dst[rep] != 0xFFFFFFFFu)
              st_dsmem_b32x4(dst[rep] + col_off, ra[2 * rep], ra[2 * rep + 1], rb[2 * rep],
                             rb[2 * rep + 1]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar0 + 8 * (kBarAccEmpty + b));  // accumulator is free again
        if (lane < C) mbar_arrive_remote(remote_bars + 8 * (kBarRecvFull + kbuf));  // rows are in place
        if (etid == 0) CH_TRACE(3, tcount);
        ++tcount;
        if (pj >= 0) {
          ok = finish_pending();
          if (!ok) break;
        }
        pj = j; ptile = tile; pbuf = kbuf; pph = bufph;
        if (++kbuf == NB) { kbuf = 0; bufph ^= 1u; }
        if (++b == 2) { b = 0; accph ^= 1u; }
      }
    }
    if (ok && pj >= 0) ok = finish_pending();
  } else if (warp >= 8) {
    // ========================================================== dequant ====
    // Four teams of four warps; team j converts the units with running number
    // j, j+4, j+8, ... into TMEM ring stage j.  Thread (c = lane % 4, g = lane / 4) of
    // quadrant q reads, for each slab of 8 packed rows, the 32-bit words at rows 2c
    // and 2c+1, byte columns 32q + 4g .. +3; byte b of the word is weight column
    // 32q + 4g + b and goes to TMEM lane 32q + 8b + g; rows (2c, 2c+1) form one bf16
    // pair = TMEM column c of that slab: the register layout of tcgen05.st.16x128b.
    const int team = (warp - 8) >> 2;
    const int q = warp & 3;
    const int c = lane & 3;
    const int g = lane >> 2;
    const uint32_t chunk = 2 * q + (g >> 2);
    const uint32_t off0 = (2 * c) * 128 + ((chunk ^ (2 * c)) << 4) + 4 * (g & 3);
    const uint32_t off1 = (2 * c + 1) * 128 + ((chunk ^ (2 * c + 1)) << 4) + 4 * (g & 3);
    const uint32_t lane_base = 32 * q;
    const int n_local = 32 * q + 4 * g;
    const uint32_t a_tmem = tmem0 + kACol0 + team * A_STAGE_COLS;
    const uint32_t a_full_bar = bar0 + 8 * (kBarReady + team);
    const uint32_t a_empty_bar = bar0 + 8 * (kBarFree + team);

    // Cursor over this team's units across the list; it runs one unit ahead of the
    // conversion so that scales and zero points (tiny, read straight from global memory)
    // are already in registers when the packed bytes arrive.
    int cj = 0, ctile = 0, cku = 0, cke = 0;
    // Position `over` units past the start of segment (j, tile); false at the end of the list.
    auto seek = [&](int j, int tile, int over) -> bool {
      while (j < NI) {
        if (tile >= P.item[j].tiles) {
          if (++j < NI) tile = first_tile(j);
          continue;
        }
        int kb, ke;
        unit_range(j, kb, ke);
        if (over < ke - kb) {
          cj = j; ctile = tile; cku = kb + over; cke = ke;
          return true;
        }
        over -= ke - kb;
        tile += NC;
      }
      cj = NI;
      return false;
    };
    auto advance = [&]() -> bool {
      cku += kAStages;
      if (cku < cke) return true;
      return seek(cj, ctile + NC, cku - cke);
    };
    uint2 sc[PLANES], zr[PLANES], sc_nx[PLANES], zr_nx[PLANES];
    auto load_sz = [&]() {
      const ChainItem& it = P.item[cj];
      const int n = ctile * kTileN + n_local;
      const bool in = n < it.N;
      const uint2* sc_ptr = reinterpret_cast<const uint2*>(it.scales);
      const uint2* zr_ptr = reinterpret_cast<const uint2*>(it.zeros);
#pragma unroll
      for (int pl = 0; pl < PLANES; ++pl) {
        const int kunit = cku + pl * it.half_units;
        const int grp = it.group_shift >= 0 ? (kunit >> it.group_shift) : (kunit / it.group_units);
        const int idx = grp * (it.N >> 2) + (n >> 2);
        sc_nx[pl] = in ? __ldg(sc_ptr + idx) : make_uint2(0u, 0u);
        if (HAS_ZERO) zr_nx[pl] = in ? __ldg(zr_ptr + idx) : make_uint2(0u, 0u);
      }
    };
    bool more = seek(0, first_tile(0), team);
    if (more) load_sz();
    int s = team;  // SW is a multiple of the team count: stages j, j+4, ... belong to team j
    uint32_t ph = 0, aph = 0;
    bool ok = true;
    while (more) {
#pragma unroll
      for (int pl = 0; pl < PLANES; ++pl) { sc[pl] = sc_nx[pl]; if (HAS_ZERO) zr[pl] = zr_nx[pl]; }
      more = advance();
      if (more) load_sz();
      ok = mbar_wait(bar0 + 8 * (kBarFullW + s), ph, abortp);
      if (!ok) break;
      const uint32_t wsrc = w_ring + s * kWStage;
      uint32_t w0[8], w1[8];
#pragma unroll
      for (int sl = 0; sl < 8; ++sl) {
        w0[sl] = lds32(wsrc + off0 + sl * 1024);
        w1[sl] = lds32(wsrc + off1 + sl * 1024);
      }
      __syncwarp();  // every lane has its words in registers
      if (lane == 0) mbar_arrive(bar0 + 8 * (kBarEmptyW + s));
      ok = mbar_wait(a_empty_bar, aph ^ 1u, abortp);
      if (!ok) break;
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
              const uint32_t Pw = prmt(w0[4 * rh + sl], w1[4 * rh + sl], 0x5410u) >> (4 * pl);
              const uint32_t Qw = prmt(w0[4 * rh + sl], w1[4 * rh + sl], 0x7632u) >> (4 * pl);
              ra[2 * sl + 0] = deq4(Pw, z2[0], s2[0]);
              ra[2 * sl + 1] = deq4(Pw >> 8, z2[1], s2[1]);
              rb[2 * sl + 0] = deq4(Qw, z2[2], s2[2]);
              rb[2 * sl + 1] = deq4(Qw >> 8, z2[3], s2[3]);
            }
            tmem_st_16x128b_x4(tmem_addr(a_tmem + pl * 32 + 16 * rh, lane_base, 0), ra);
            tmem_st_16x128b_x4(tmem_addr(a_tmem + pl * 32 + 16 * rh, lane_base + 16, 0), rb);
          }
        }
      } else {
        const float sf[4] = {bf16lo_f32(sc[0].x), bf16hi_f32(sc[0].x), bf16lo_f32(sc[0].y),
                             bf16hi_f32(sc[0].y)};
        float cz[4];
        if (HAS_ZERO) {
          cz[0] = 8388608.0f + bf16lo_f32(zr[0].x); cz[1] = 8388608.0f + bf16hi_f32(zr[0].x);
          cz[2] = 8388608.0f + bf16lo_f32(zr[0].y); cz[3] = 8388608.0f + bf16hi_f32(zr[0].y);
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
          tmem_st_16x128b_x4(tmem_addr(a_tmem + 16 * rh, lane_base, 0), ra);
          tmem_st_16x128b_x4(tmem_addr(a_tmem + 16 * rh, lane_base + 16, 0), rb);
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_full_bar);
      aph ^= 1u;
      s += kAStages;
      if (s >= SW) { s -= SW; ph ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem0, 512);
  if (threadIdx.x == 0) {
    if (abort_flag) atomicExch(P.status, DXB_ERR_KERNEL_TIMEOUT);
    // The last CTA to get here puts the completion counts back to zero for the next launch.
    __threadfence();
    if (atomicAdd(P.exits, 1) == static_cast<int>(gridDim.x) - 1) {
      for (int j = 0; j < NI; ++j) P.done[j] = 0;
      *P.exits = 0;
    }
  }
  // Peers may still be writing this CTA's receive buffers or arriving on its barriers.
  cluster_sync_all();
}

// ------------------------------------------------------------------ host side
struct ChainPlan {
  int cluster = 0, clusters = 0, w_stages = 0, x_stage_bytes = 0, recv_off = 0, recv_bytes = 0,
      recv_bufs = 1;
  size_t smem_bytes = 0;
  size_t total_bytes = 0;
  int NU[kMaxChain], U[kMaxChain], tiles[kMaxChain], rot[kMaxChain], need_done[kMaxChain],
      rows_per[kMaxChain];
};

constexpr size_t kChainExitsOff = 64;   // inside the status block: CTAs that have finished
constexpr size_t kChainDoneOff = 128;  // inside the status block: done[kMaxChain]

// Largest number of C-CTA clusters of the chain kernel that are resident together.
template <int BITS, bool HAS_ZERO>
static int resident_clusters(int C) {
  auto kernel = wq_chain_tc<BITS, HAS_ZERO>;
  static thread_local int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemBudget + 1024) != cudaSuccess)
      return 0;
    attr_dev = dev;
  }
  static thread_local int cache_dev = -1;
  static thread_local int cache[9];
  if (cache_dev != dev) {
    for (int i = 0; i < 9; ++i) cache[i] = -1;
    cache_dev = dev;
  }
  if (cache[C] >= 0) return cache[C];
  cudaLaunchConfig_t qcfg = {};
  qcfg.gridDim = dim3(C);
  qcfg.blockDim = dim3(kThreads);
  qcfg.dynamicSmemBytes = kSmemBudget + 1024;
  cudaLaunchAttribute qattr[1];
  qattr[0].id = cudaLaunchAttributeClusterDimension;
  qattr[0].val.clusterDim.x = C;
  qattr[0].val.clusterDim.y = 1;
  qattr[0].val.clusterDim.z = 1;
  qcfg.attrs = qattr;
  qcfg.numAttrs = 1;
  int resident = 0;
  if (cudaOccupancyMaxActiveClusters(&resident, kernel, &qcfg) != cudaSuccess) {
    cudaGetLastError();
    resident = 0;
  }
  cache[C] = resident;
  return resident;
}

static long long* g_chain_trace = nullptr;

static int chain_cluster_override() {
  static const int v = [] {
    const char* e = getenv("DEXTER_B200_CHAIN_CLUSTER");
    return e ? atoi(e) : 0;
  }();
  return v;
}

template <int BITS, bool HAS_ZERO>
static int plan_chain(const dxb_chain_item* items, int n, int max_ctas, ChainPlan* pl) {
  if (items == nullptr) return DXB_ERR_NULL;
  if (n < 1 || n > kMaxChain) return DXB_ERR_UNSUPPORTED;
  // Cluster size: the one that keeps most CTAs resident (4 before 8 before 2 on a tie).
  const int cands[3] = {4, 8, 2};
  int best_c = 0, best_ctas = 0;
  for (int i = 0; i < 3; ++i) {
    const int C = cands[i];
    if (chain_cluster_override() && chain_cluster_override() != C) continue;
    int nc = resident_clusters<BITS, HAS_ZERO>(C);
    if (max_ctas > 0 && nc > max_ctas / C) nc = max_ctas / C;
    if (nc * C > best_ctas) { best_ctas = nc * C; best_c = C; }
  }
  if (best_c == 0) return DXB_ERR_UNSUPPORTED;
  const int C = best_c;
  pl->cluster = C;
  pl->clusters = best_ctas / C;
  const int planes = BITS == 4 ? 2 : 1;
  int rot = 0, rows_max = 1;
  pl->x_stage_bytes = 0;
  for (int j = 0; j < n; ++j) pl->need_done[j] = 0;
  for (int j = 0; j < n; ++j) {
    const dxb_chain_item& it = items[j];
    if (!it.x || !it.qweight || !it.scales || !it.out) return DXB_ERR_NULL;
    if (it.M <= 0 || it.N <= 0 || it.K <= 0 || it.group_size <= 0) return DXB_ERR_SHAPE;
    if (it.K % it.group_size || it.ldx < it.K || it.ldo < it.N) return DXB_ERR_SHAPE;
    if ((it.zeros != nullptr) != HAS_ZERO) return DXB_ERR_UNSUPPORTED;
    if (it.depends_on >= j || it.depends_on < -1) return DXB_ERR_SHAPE;
    if (!tc_supported(it.M, it.N, it.K, it.group_size, BITS)) return DXB_ERR_UNSUPPORTED;
    const bool aligned = (reinterpret_cast<uintptr_t>(it.x) % 16 == 0) && (it.ldx % 8 == 0) &&
                         (reinterpret_cast<uintptr_t>(it.qweight) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(it.scales) % 16 == 0) &&
                         (it.zeros == nullptr || reinterpret_cast<uintptr_t>(it.zeros) % 16 == 0) &&
                         (it.bias == nullptr || reinterpret_cast<uintptr_t>(it.bias) % 8 == 0) &&
                         (reinterpret_cast<uintptr_t>(it.out) % 16 == 0) && (it.ldo % 8 == 0) &&
                         (BITS != 4 || (it.K / 2) % 8 == 0);
    if (!aligned) return DXB_ERR_UNSUPPORTED;
    const int rows = BITS == 4 ? it.K / 2 : it.K;
    pl->NU[j] = ((it.M + 15) / 16) * 16;
    pl->U[j] = rows / kUnitRows;
    if (pl->U[j] < C) return DXB_ERR_UNSUPPORTED;  // every CTA of a cluster needs a K unit
    pl->tiles[j] = (it.N + kTileN - 1) / kTileN;
    pl->rot[j] = rot;
    rot = (rot + pl->tiles[j]) % pl->clusters;
    pl->rows_per[j] = (it.M + C - 1) / C;
    if (pl->rows_per[j] > rows_max) rows_max = pl->rows_per[j];
    if (it.depends_on >= 0) pl->need_done[it.depends_on] = 1;
    const int xb = planes * pl->NU[j] * 128;
    if (xb > pl->x_stage_bytes) pl->x_stage_bytes = xb;
  }
  pl->total_bytes = kStatusBytes;
  // Shared memory: four activation stages, the receive buffers (C x rows_per rows of 128
  // fp32), and as deep a packed-weight ring (a multiple of four stages) as still fits.
  const int recv_bytes = C * rows_max * kTileN * 4;
  int w_stages = 0, bufs = 2;
  for (; bufs >= 1; --bufs) {  // two receive buffers if a weight ring of four stages still fits
    w_stages = (kSmemBudget - kAStages * pl->x_stage_bytes - bufs * recv_bytes) / kWStage;
    w_stages = (w_stages / kAStages) * kAStages;
    if (w_stages >= kAStages) break;
  }
  if (bufs < 1) return DXB_ERR_UNSUPPORTED;
  if (w_stages > kMaxWStages) w_stages = kMaxWStages;
  pl->w_stages = w_stages;
  pl->recv_bytes = recv_bytes;
  pl->recv_bufs = bufs;
  pl->recv_off = w_stages * kWStage + kAStages * pl->x_stage_bytes;
  pl->smem_bytes = static_cast<size_t>(pl->recv_off) + static_cast<size_t>(bufs) * recv_bytes + 1024;
  return DXB_OK;
}

template <int BITS, bool HAS_ZERO>
static int launch_chain(const dxb_chain_item* items, int n, const ChainPlan& pl, void* workspace,
                        cudaStream_t stream) {
  static_assert(kChainDoneOff + kMaxChain * sizeof(int) <= kStatusBytes, "status block too small");
  static_assert(kChainExitsOff + sizeof(int) <= kChainDoneOff, "status block layout");
  ChainParams P;
  memset(&P, 0, sizeof(P));
  uint8_t* wsb = static_cast<uint8_t*>(workspace);
  P.status = reinterpret_cast<int*>(wsb);
  P.done = reinterpret_cast<int*>(wsb + kChainDoneOff);
  P.exits = reinterpret_cast<int*>(wsb + kChainExitsOff);
  P.n = n;
  P.w_stages = pl.w_stages;
  P.x_stage_bytes = pl.x_stage_bytes;
  P.recv_off = pl.recv_off;
  P.recv_bytes = pl.recv_bytes;
  P.recv_bufs = pl.recv_bufs;
  P.cluster = pl.cluster;
  P.trace = g_chain_trace;
  for (int j = 0; j < n; ++j) {
    const dxb_chain_item& it = items[j];
    const int rows = BITS == 4 ? it.K / 2 : it.K;
    bool ok;
    {
      const uint64_t dims[2] = {static_cast<uint64_t>(it.N), static_cast<uint64_t>(rows)};
      const uint64_t strides[1] = {static_cast<uint64_t>(it.N)};
      const uint32_t box[2] = {kTileN, kUnitRows};
      ok = make_map(&P.tm_q[j], it.qweight, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, dims, strides, box,
                    CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (BITS == 4) {
      const uint64_t dims[3] = {static_cast<uint64_t>(it.K / 2), static_cast<uint64_t>(it.M), 2};
      const uint64_t strides[2] = {static_cast<uint64_t>(it.ldx) * 2,
                                   static_cast<uint64_t>(it.K / 2) * 2};
      const uint32_t box[3] = {64, static_cast<uint32_t>(pl.NU[j]), 2};
      ok = ok && make_map(&P.tm_x[j], it.x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
      const uint64_t dims[2] = {static_cast<uint64_t>(it.K), static_cast<uint64_t>(it.M)};
      const uint64_t strides[1] = {static_cast<uint64_t>(it.ldx) * 2};
      const uint32_t box[2] = {64, static_cast<uint32_t>(pl.NU[j])};
      ok = ok && make_map(&P.tm_x[j], it.x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (!ok) return DXB_ERR_TENSORMAP;
    ChainItem& ci = P.item[j];
    ci.scales = static_cast<const __nv_bfloat16*>(it.scales);
    ci.zeros = static_cast<const __nv_bfloat16*>(it.zeros);
    ci.bias = static_cast<const __nv_bfloat16*>(it.bias);
    ci.out = static_cast<__nv_bfloat16*>(it.out);
    ci.ldo = it.ldo;
    ci.M = it.M; ci.N = it.N; ci.NU = pl.NU[j];
    ci.U = pl.U[j];
    ci.tiles = pl.tiles[j];
    ci.half_units = BITS == 4 ? (it.K / 2) / kUnitRows : 0;
    ci.group_units = it.group_size / kUnitRows;
    ci.group_shift = -1;
    for (int b = 0; b < 20; ++b) if ((1 << b) == ci.group_units) ci.group_shift = b;
    ci.x_bytes = (BITS == 4 ? 2 : 1) * pl.NU[j] * 128;
    ci.dep = it.depends_on;
    ci.rot = pl.rot[j];
    ci.need_done = pl.need_done[j];
    ci.rows_per = pl.rows_per[j];
    ci.rows_inv = (65536 + ci.rows_per - 1) / ci.rows_per;
  }

  auto kernel = wq_chain_tc<BITS, HAS_ZERO>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.clusters * pl.cluster);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = pl.cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, P) != cudaSuccess) {
    cudaGetLastError();
    return DXB_ERR_CUDA;
  }
  return cudaGetLastError() == cudaSuccess ? DXB_OK : DXB_ERR_CUDA;
}

template <int BITS, bool HAS_ZERO>
static int run_chain(const dxb_chain_item* items, int n, void* workspace, size_t workspace_bytes,
                     int max_ctas, cudaStream_t stream, size_t* need_only) {
  ChainPlan pl;
  const int rc = plan_chain<BITS, HAS_ZERO>(items, n, max_ctas, &pl);
  if (need_only) {
    *need_only = rc == DXB_OK ? pl.total_bytes : 0;
    return rc;
  }
  if (rc != DXB_OK) return rc;
  if (workspace == nullptr || workspace_bytes < pl.total_bytes) return DXB_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) % 256) return DXB_ERR_WORKSPACE;
  return launch_chain<BITS, HAS_ZERO>(items, n, pl, workspace, stream);
}

static int dispatch_chain(int bits, const dxb_chain_item* items, int n, void* workspace,
                          size_t workspace_bytes, int max_ctas, cudaStream_t stream,
                          size_t* need_only) {
  if (bits != 4 && bits != 8) return DXB_ERR_BITS;
  if (items == nullptr) return DXB_ERR_NULL;
  if (n < 1 || n > kMaxChain) return DXB_ERR_UNSUPPORTED;
  const bool has_zero = items[0].zeros != nullptr;
  if (bits == 4)
    return has_zero ? run_chain<4, true>(items, n, workspace, workspace_bytes, max_ctas, stream, need_only)
                    : run_chain<4, false>(items, n, workspace, workspace_bytes, max_ctas, stream, need_only);
  return has_zero ? run_chain<8, true>(items, n, workspace, workspace_bytes, max_ctas, stream, need_only)
                  : run_chain<8, false>(items, n, workspace, workspace_bytes, max_ctas, stream, need_only);
}

}  // namespace dx

extern "C" {

#ifdef DXB_TRACE
void dxb_debug_set_chain_trace(void* ptr) { dx::g_chain_trace = static_cast<long long*>(ptr); }
#endif

size_t dxb_chain_workspace_bytes(int bits, const dxb_chain_item* items, int n_items, int max_ctas) {
  size_t need = 0;
  dx::dispatch_chain(bits, items, n_items, nullptr, 0, max_ctas, nullptr, &need);
  return need;
}

int dxb_wq_gemm_chain(int bits, const dxb_chain_item* items, int n_items, void* workspace,
                      size_t workspace_bytes, int max_ctas, void* cuda_stream) {
  return dx::dispatch_chain(bits, items, n_items, workspace, workspace_bytes, max_ctas,
                            static_cast<cudaStream_t>(cuda_stream), nullptr);
}

}  // extern "C"
