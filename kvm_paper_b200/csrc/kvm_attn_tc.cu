// Block attention of the prefill on the Blackwell tensor cores (tcgen05 + tensor memory), head_dim 128.
//
// One CTA = NQ query tiles of 128 rows (NQ = 2: a whole 256-row slice of a query block) of one
// (batch, q-head).  Keys/values are consumed in tiles of 64 rows shared by the query tiles: two window tiles,
// then the memory version of the block (rows gathered from the row pool through the version's index table),
// then the rest of the sliding window up to the diagonal.
//
//   softmax warpgroups (NQ x 4 warps)  one query row per thread (= one tensor-memory lane): tcgen05.ld of
//               the score tile, scale by the segment's temperature, mask, exp2, row sum, bf16 P written with
//               tcgen05.st over the columns of the score tile it came from (P never touches shared memory).
//               The running maximum is only raised (and O in tensor memory rescaled with tcgen05.ld/st, 16
//               columns at a time) when a tile exceeds it by more than 2^8.  At the end: O / l as bf16 into
//               the query tile's operand buffer, two TMA stores.
//   loader warps (4)   tile t is loaded by loader t % 4 into stage t % 4: tiled TMA for window tiles, 16-byte
//               cp.async through the version table for memory tiles (128B-swizzled operand layouts, fence to
//               the async proxy, mbarrier arrive); four tiles are in flight.  Query tiles and the two leading
//               window tiles are issued by thread 0 before the plan entry is read.
//   MMA warps (NQ)   one thread per query tile issues tcgen05.mma:  S = Q K^T into tensor memory (two S buffers
//               per query tile, so the next score tile is computed while the current one is in softmax),
//               O += P V with P as the tensor-memory A operand
// Tensor memory: NQ x 2 score buffers of 64 columns (P aliases their first 32), NQ output accumulators of 128.
// Every mbarrier wait is bounded; on expiry the CTA records a status code, falls through to the common
// exit, frees its tensor memory and returns.
#include "kvm_common.cuh"
#include "kvm_tc.cuh"
#include "kvm_tma_host.cuh"

namespace kvm {

namespace {

constexpr int BM = 128;  // rows per query tile
constexpr int BN = 64;   // keys per tile
constexpr int HD = 128;  // head dim
constexpr int kStages = 4;
constexpr int kLoaders = 4;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// Tile order of a CTA: `lead` window tiles (they arrive by TMA right after the CTA starts, while the first memory
// tiles still wait for the plan entry, the version table and the row gather), then the memory tiles, then the
// remaining window tiles.  `lead` is at most the number of window tiles that every query tile of the CTA uses,
// so each query tile still consumes a prefix of the order.
constexpr int kLeadWindowTiles = 2;

template <int NQ>
struct Cfg {
  static constexpr int kSoftmaxWarps = NQ * 4;
  static constexpr int kThreads = (kSoftmaxWarps + kLoaders + NQ) * 32;
  static constexpr int kMmaWarp = kSoftmaxWarps + kLoaders;    // first of NQ MMA-issuing warps
  static constexpr uint32_t kTmemCols = NQ == 2 ? 512 : 256;
  static constexpr uint32_t kColO = NQ * 128;                  // first column of the output accumulators
  static constexpr uint32_t kOffQ = 0;                         // NQ x 2 x [128][64] bf16
  static constexpr uint32_t kOffK = NQ * 32768;                // kStages x 2 x [64][64]
  static constexpr uint32_t kOffV = kOffK + kStages * 16384;   // kStages x 2 x [64 keys][64]
  static constexpr uint32_t kOffBar = kOffV + kStages * 16384;
  static constexpr uint32_t kSmemBytes = kOffBar + 256;
};

struct Bars {
  uint64_t q_full[2], kv_full[kStages], kv_empty[kStages], s_full[2][2], p_full[2][2], pv_done[2], o_final[2], o_ready[2];
  uint32_t tmem_base;
};

// All 32 lanes wait; the result is made uniform over the warp so that no lane leaves a loop alone.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity) {
  const bool ok = tc::mbar_wait(bar, parity);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Geometry of one CTA, computed identically by every role.
template <int NQ>
struct Slice {
  int b, hq, hkv, S, n_mem_tiles, n_max, lead;
  long long q0, bb, q_end_all;
  long long q_end[NQ];
  int n_tiles[NQ];
  const bf16* mk;
  const bf16* mv;
  const int* midx;
  // per-query-tile values picked with compile-time indices, so that the slice stays in registers
  __device__ __forceinline__ int tiles_of(int qi) const { return (NQ == 1 || qi == 0) ? n_tiles[0] : n_tiles[NQ - 1]; }
  __device__ __forceinline__ long long q_end_of(int qi) const { return (NQ == 1 || qi == 0) ? q_end[0] : q_end[NQ - 1]; }
};

// ------------------------------------------------------------------------------------------ loaders
// The q, k, v inputs as 4-D tensors [batch][head][token][D] (any strides): boxes of 64 elements x 128 tokens
// (queries) or 64 tokens (keys, values) land in the 128-byte-swizzled operand layout.
struct AttnMaps {
  CUtensorMap q, k, v, o;  // o: the output [B, T, Hq, D] with boxes of 64 elements x 128 tokens
  int q_head_inner, kv_head_inner;  // the head dimension has the smaller stride ([B,T,H,D] storage): it comes second
  // head-sharded prefill that gathers by itself: `o` and `o_peer` describe every rank's [B, T, n_ranks*Hq, D] buffer
  // (this rank's first), the CTA stores its tile into each at head `h_off + hq`
  CUtensorMap o_peer[7];
  int n_peer, h_off;
};
// box at (element x, token t, head h, batch b) of a tensor whose dimensions are ordered by stride
__device__ __forceinline__ void attn_tma(void* dst, const CUtensorMap* m, bool head_inner, int x, int t, int h, int b,
                                         uint64_t* bar) {
  if (head_inner) tc::tma_load_4d(dst, m, x, h, t, b, bar);
  else tc::tma_load_4d(dst, m, x, t, h, b, bar);
}

// Query tiles and window tiles are contiguous token ranges: one thread issues tiled TMA copies (two per operand,
// one per 64-element half of the head dimension) that signal the destination's barrier with their byte count.
// Rows past the end of the sequence read as zeros; rows past the query block are real tokens that the causal
// mask hides.
// One thread: query tile qi (128 tokens from `qs`) -> its operand buffer.
template <int NQ>
__device__ __forceinline__ void issue_query_tile(unsigned char* smem, Bars* bars, const AttnMaps* maps, int b, int hq,
                                                 int qi, int qs) {
  unsigned char* dQ = smem + Cfg<NQ>::kOffQ + qi * 32768;
  tc::mbar_arrive_expect_tx(&bars->q_full[qi], 2u * BM * 128u);
  attn_tma(dQ, &maps->q, maps->q_head_inner != 0, 0, qs, hq, b, &bars->q_full[qi]);
  attn_tma(dQ + 16384, &maps->q, maps->q_head_inner != 0, 64, qs, hq, b, &bars->q_full[qi]);
}
// One thread: 64 window tokens from `r0` (keys and values) -> stage `stage`.
template <int NQ>
__device__ __forceinline__ void issue_window_tile(unsigned char* smem, Bars* bars, const AttnMaps* maps, int b, int hkv,
                                                  int stage, int r0) {
  unsigned char* dK = smem + Cfg<NQ>::kOffK + stage * 16384;
  unsigned char* dV = smem + Cfg<NQ>::kOffV + stage * 16384;
  tc::mbar_arrive_expect_tx(&bars->kv_full[stage], 4u * BN * 128u);
  const bool hi = maps->kv_head_inner != 0;
  attn_tma(dK, &maps->k, hi, 0, r0, hkv, b, &bars->kv_full[stage]);
  attn_tma(dK + 8192, &maps->k, hi, 64, r0, hkv, b, &bars->kv_full[stage]);
  attn_tma(dV, &maps->v, hi, 0, r0, hkv, b, &bars->kv_full[stage]);
  attn_tma(dV + 8192, &maps->v, hi, 64, r0, hkv, b, &bars->kv_full[stage]);
}

// Loader `lw` brings the key/value tiles t = lw, lw+4, ... into stage lw, except the query tiles and the leading
// window tiles, which thread 0 issues when the CTA starts (they need nothing from the plan).  Memory tiles are
// gathered row by row through the version table with 16-byte cp.async.  Returns false if a bounded wait expired.
template <int NQ>
__device__ __forceinline__ bool loader_role(const Slice<NQ>& sl, unsigned char* smem, Bars* bars, int lw, int lane,
                                            const AttnMaps* maps) {
  using CF = Cfg<NQ>;
  const int stage = lw;
  unsigned char* dK = smem + CF::kOffK + stage * 16384;
  unsigned char* dV = smem + CF::kOffV + stage * 16384;
  // lane -> fixed 16-byte column chunk cc and row parity; iteration `it` covers rows 2*it and 2*it+1
  const int cc = lane & 15, rh = lane >> 4;
  const uint32_t col_off = (uint32_t)(cc >> 3) * 8192u;
  for (int t = lw; t < sl.n_max; t += kLoaders) {
    if (t < sl.lead) continue;  // issued when the CTA started
    if (t >= kStages && !warp_wait(&bars->kv_empty[stage], ((t / kStages) - 1) & 1)) return false;
    const bool is_mem = t < sl.lead + sl.n_mem_tiles;
    if (!is_mem) {
      if (lane == 0) issue_window_tile<NQ>(smem, bars, maps, sl.b, sl.hkv, stage, (int)(sl.bb + (long long)(t - sl.n_mem_tiles) * BN));
      __syncwarp();
      continue;
    }
    const int row0 = (t - sl.lead) * BN;
    const int i0 = row0 + lane < sl.S ? __ldg(sl.midx + row0 + lane) : 0;
    const int i1 = row0 + 32 + lane < sl.S ? __ldg(sl.midx + row0 + 32 + lane) : 0;
#pragma unroll
    for (int it = 0; it < BN / 2; ++it) {
      const int r = it * 2 + rh;
      const int a0 = __shfl_sync(0xffffffffu, it < 16 ? i0 : i1, r & 31);
      const bool ok = row0 + r < sl.S;
      const uint32_t off = col_off + (uint32_t)(r * 128) + (uint32_t)((((cc & 7) ^ (r & 7)) & 7) << 4);
      const size_t src = (size_t)a0 * HD + cc * 8;
      cp_async16(dK + off, sl.mk + src, ok ? 16 : 0);
      cp_async16(dV + off, sl.mv + src, ok ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();       // this warp's tile has landed
    tc::fence_proxy_async();  // generic-proxy writes -> visible to the tensor core's operand reads
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&bars->kv_full[stage]);
  }
  return true;
}

// ------------------------------------------------------------------------------------------ MMA issue
// One thread per query tile issues that tile's MMAs (a single thread issuing for both query tiles spent
// more cycles issuing than the tensor core needs to execute).  Order: QK of tiles 0 and 1, then per tile t:
// P V (as the softmax delivers P), release of the stage, QK of tile t+2.  A stage is released by every
// issuer: one that does not use a tile (the causal range of its query tile ends earlier) still arrives
// on the stage's barrier, after the tile has landed, so that arrivals stay in step with the stage's uses.
template <int NQ>
__device__ __forceinline__ bool mma_role(const Slice<NQ>& sl, unsigned char* smem, Bars* bars, uint32_t tmem, int qi) {
  using CF = Cfg<NQ>;
  constexpr uint32_t idesc_qk = tc::make_idesc(BM, BN, 0, 0);
  constexpr uint32_t idesc_pv = tc::make_idesc(BM, HD, 0, 1);
  const uint32_t sQ = tc::smem_u32(smem + CF::kOffQ), sK = tc::smem_u32(smem + CF::kOffK);
  const uint32_t sV = tc::smem_u32(smem + CF::kOffV);
  // descriptors differ only in their 14-bit start-address field: build each base once, then add offsets
  const uint64_t dQ = tc::make_desc(sQ, 16, 1024) + (uint64_t)((qi * 32768) >> 4), dK = tc::make_desc(sK, 16, 1024);
  const uint64_t dV = tc::make_desc(sV, 8192, 1024);
  const int nt = sl.tiles_of(qi);
  auto issue_qk = [&](int t) {
    const int stage = t % kStages, sbuf = t & 1;
    const uint32_t d = tmem + (uint32_t)((qi * 2 + sbuf) * BN);
    const uint64_t db0 = dK + (uint64_t)((stage * 16384) >> 4);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const uint64_t da = dQ + (uint64_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
      const uint64_t db = db0 + (uint64_t)(((ks >> 2) * 8192 + (ks & 3) * 32) >> 4);
      tc::mma_ss(d, da, db, idesc_qk, ks > 0);
    }
    tc::mma_commit(&bars->s_full[qi][sbuf]);
  };
  if (nt > 0 && !tc::mbar_wait(&bars->q_full[qi], 0)) return false;
  for (int t = 0; t < 2 && t < nt; ++t) {
    if (!tc::mbar_wait(&bars->kv_full[t % kStages], 0)) return false;
    tc::tc_fence_after_sync();
    issue_qk(t);
  }
  for (int t = 0; t < sl.n_max; ++t) {
    const int stage = t % kStages;
    if (t < nt) {
      // (one barrier per score buffer: a softmax warp that is a tile ahead of its neighbours arrives on the other one
      // and cannot complete this tile's phase in their place)
      if (!tc::mbar_wait(&bars->p_full[qi][t & 1], (t >> 1) & 1)) return false;
      tc::tc_fence_after_sync();
      const uint64_t db0 = dV + (uint64_t)((stage * 16384) >> 4);
      // P (bf16) lies in the first 32 columns of the score buffer it was computed from: 8 columns per k-step
      const uint32_t aP = tmem + (uint32_t)((qi * 2 + (t & 1)) * BN);
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks)
        tc::mma_ts(tmem + CF::kColO + qi * 128, aP + (uint32_t)(ks * 8), db0 + (uint64_t)((ks * 2048) >> 4), idesc_pv,
                   (t > 0) || (ks > 0));
      tc::mma_commit(&bars->pv_done[qi]);
      tc::mma_commit(&bars->kv_empty[stage]);
      // The epilogue waits on a barrier of its own: the softmax only waits on pv_done before a rescale, so at
      // the end of the tile loop pv_done may be two phases behind, which a parity wait cannot tell from done.
      if (t == nt - 1) tc::mma_commit(&bars->o_final[qi]);
    } else {
      if (!tc::mbar_wait(&bars->kv_full[stage], (t / kStages) & 1)) return false;
      tc::mbar_arrive(&bars->kv_empty[stage]);
    }
    if (t + 2 < nt) {
      if (!tc::mbar_wait(&bars->kv_full[(t + 2) % kStages], ((t + 2) / kStages) & 1)) return false;
      tc::tc_fence_after_sync();
      issue_qk(t + 2);
    }
  }
  return true;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// ------------------------------------------------------------------------------------------ softmax
// One query row per thread of warpgroup qi.  Returns false if a bounded wait expired.
template <int NQ>
__device__ __forceinline__ bool softmax_role(const Slice<NQ>& sl, const LayerDev& L, unsigned char* smem, Bars* bars,
                                             uint32_t tmem, int qi, int row, int wq, int lane, float sm_scale,
                                             const AttnMaps* maps) {
  using CF = Cfg<NQ>;
  const int nt = sl.tiles_of(qi);
  if (nt <= 0) return true;
  // positions relative to the first window token (32-bit: the window is a few blocks long)
  const int qs_rel = (int)(sl.q0 - sl.bb) + qi * BM, q_rel = qs_rel + row;
  const int S = sl.S, nm = sl.n_mem_tiles, lead = sl.lead;
  const uint32_t lane_addr = tmem + ((uint32_t)(wq * 32) << 16);
  const uint32_t col_o = CF::kColO + qi * 128;
  const float scale_mem = sm_scale * L.state_temp[sl.hq] * kLog2e;
  const float scale_win = sm_scale * L.front_temp[sl.hq] * kLog2e;
  float m_run = -INFINITY, l_run = 0.f;
  for (int t = 0; t < nt; ++t) {
    const int sbuf = t & 1;
    if (!warp_wait(&bars->s_full[qi][sbuf], (t >> 1) & 1)) return false;
    tc::tc_fence_after_sync();
    uint32_t sr[2][32];
    tc::tmem_ld32(lane_addr + (uint32_t)((qi * 2 + sbuf) * BN), sr[0]);
    tc::tmem_ld32(lane_addr + (uint32_t)((qi * 2 + sbuf) * BN + 32), sr[1]);
    tc::tmem_ld_wait();
    const bool is_mem = t >= lead && t < lead + nm;
    const int base = (is_mem ? t - lead : (t < lead ? t : t - nm)) * BN;  // first key of the tile within its segment
    const float sc = is_mem ? scale_mem : scale_win;
    // keys [0, n_ok) of this tile are visible to this row (memory: rows below S; window: causal)
    const int n_ok = max(0, min(BN, (is_mem ? S : q_rel + 1) - base));
    const bool tile_masked = base + BN > (is_mem ? S : qs_rel + 1);  // uniform over the warpgroup
    if (tile_masked) {
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (i >= n_ok) sr[i >> 5][i & 31] = 0xff800000u;  // -inf
    }
    float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      tm0 = max3(tm0, __uint_as_float(sr[0][i]), __uint_as_float(sr[0][i + 1]));
      tm1 = max3(tm1, __uint_as_float(sr[1][i]), __uint_as_float(sr[1][i + 1]));
    }
    const float tmax = fmaxf(tm0, tm1) * sc;  // sc > 0
    const bool need = tmax > m_run + kRescaleThreshold || (m_run == -INFINITY && tmax > -INFINITY);
    const bool warp_need = __any_sync(0xffffffffu, need);
    if (warp_need) {
      // the running output may only be touched between P V of tile t-1 (complete) and of tile t (not yet issued:
      // it waits for this warp's arrival below)
      if (t > 0 && !warp_wait(&bars->pv_done[qi], (t - 1) & 1)) return false;
      const float m_new = fmaxf(m_run, tmax);
      const float alpha = (m_run == -INFINITY) ? 0.f : ex2(m_run - m_new);
      l_run *= alpha;
      if (t > 0) {  // rescale the running output of this warp's 32 rows in tensor memory
        tc::tc_fence_after_sync();
#pragma unroll
        for (int cb = 0; cb < HD / 16; ++cb) {  // 16 columns at a time: the scores of the tile stay in registers
          uint32_t o[16];
          tc::tmem_ld16(lane_addr + col_o + cb * 16, o);
          tc::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float2 r = __fmul2_rn(make_float2(__uint_as_float(o[i]), __uint_as_float(o[i + 1])), make_float2(alpha, alpha));
            o[i] = __float_as_uint(r.x);
            o[i + 1] = __float_as_uint(r.y);
          }
          tc::tmem_st16(lane_addr + col_o + cb * 16, o);
        }
        tc::tmem_st_wait();
      }
      m_run = m_new;
    }
    const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
    float2 ls = make_float2(0.f, 0.f);
    const float2 sc2 = make_float2(sc, sc), nm2 = make_float2(neg_m, neg_m);
    // P replaces the scores it came from (all 64 columns of this row are in registers): the A operand of P V,
    // written in two halves of 16 columns (32 keys) each
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        // two keys per instruction: the packed fp32 forms of the multiply-add and of the add
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[half][e * 2]), __uint_as_float(sr[half][e * 2 + 1])), sc2, nm2);
        const float2 p = make_float2(ex2(x.x), ex2(x.y));
        ls = __fadd2_rn(ls, p);
        pk[e] = pack_bf16(p.x, p.y);
      }
      tc::tmem_st16(lane_addr + (uint32_t)((qi * 2 + sbuf) * BN + half * 16), pk);
    }
    l_run += ls.x + ls.y;
    tc::tmem_st_wait();
    tc::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&bars->p_full[qi][sbuf]);
  }
  // epilogue: O / l -> bf16 -> the query tile's operand buffer (all QK of this tile have completed), in the
  // 128-byte-swizzled layout of a [128 tokens][64] box per half of the head dimension -> two TMA stores into
  // [B, T, Hq*D]; tokens past the end of the sequence are clipped by the tensor map
  if (!warp_wait(&bars->o_final[qi], 0)) return false;
  tc::tc_fence_after_sync();
  const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
  unsigned char* dO = smem + CF::kOffQ + qi * 32768;
  // (64 columns per round trip to tensor memory: the score registers of the loop are free by now)
#pragma unroll
  for (int hb = 0; hb < HD / 64; ++hb) {
    uint32_t o[2][32];
    tc::tmem_ld32(lane_addr + col_o + hb * 64, o[0]);
    tc::tmem_ld32(lane_addr + col_o + hb * 64 + 32, o[1]);
    tc::tmem_ld_wait();
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {  // 16-byte chunk c8 of this half's 128-byte row
      const uint32_t* oo = &o[c8 >> 2][(c8 & 3) * 8];
      uint4 o8;
      o8.x = pack_bf16(__uint_as_float(oo[0]) * inv, __uint_as_float(oo[1]) * inv);
      o8.y = pack_bf16(__uint_as_float(oo[2]) * inv, __uint_as_float(oo[3]) * inv);
      o8.z = pack_bf16(__uint_as_float(oo[4]) * inv, __uint_as_float(oo[5]) * inv);
      o8.w = pack_bf16(__uint_as_float(oo[6]) * inv, __uint_as_float(oo[7]) * inv);
      *reinterpret_cast<uint4*>(dO + hb * 16384 + row * 128 + (((c8 ^ (row & 7)) & 7) << 4)) = o8;
    }
  }
  tc::fence_proxy_async();  // generic-proxy writes -> visible to the TMA store
  __syncwarp();
  if (lane == 0) tc::mbar_arrive(&bars->o_ready[qi]);
  if (wq == 0) {
    if (!warp_wait(&bars->o_ready[qi], 0)) return false;
    if (lane == 0) {
      const int qs = (int)(sl.q0 + (long long)qi * BM);
      const int hh = sl.hq + maps->h_off;
      tc::tma_store_4d(&maps->o, dO, 0, hh, qs, sl.b);
      tc::tma_store_4d(&maps->o, dO + 16384, 64, hh, qs, sl.b);
      // the same tile into the other ranks' buffers (peer memory over NVLink: the gather of the outputs rides on the
      // copy engine while the other CTAs compute)
      for (int pr = 0; pr < maps->n_peer; ++pr) {
        tc::tma_store_4d(&maps->o_peer[pr], dO, 0, hh, qs, sl.b);
        tc::tma_store_4d(&maps->o_peer[pr], dO + 16384, 64, hh, qs, sl.b);
      }
      tc::bulk_commit_group();
      tc::bulk_wait_group_read0();  // shared memory must outlive the copy
    }
    __syncwarp();
  }
  return true;
}

}  // namespace

template <int NQ>
__global__ void __launch_bounds__(Cfg<NQ>::kThreads, 1)
kvm_attn_prefill_tc_kernel(LayerDev L, long long T, Tensor4 q, Tensor4 k, Tensor4 v,
                           const kvm_update_plan* __restrict__ plan, const bf16* __restrict__ pool_k,
                           const bf16* __restrict__ pool_v, long long pool_rows, const int* __restrict__ ver_idx,
                           long long ver_rows, bf16* __restrict__ out, int ctas_per_block, float sm_scale,
                           int* __restrict__ status, const __grid_constant__ AttnMaps maps) {
  using CF = Cfg<NQ>;
  extern __shared__ __align__(1024) unsigned char smem[];
  if (*status != 0) return;  // an earlier kernel of this prefill gave up: the version tables are not to be trusted
  Bars* bars = reinterpret_cast<Bars*>(smem + CF::kOffBar);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = L.C;

  Slice<NQ> sl;
  const int xi = gridDim.x - 1 - blockIdx.x;  // later (heavier) slices first
  const int j = xi / ctas_per_block;
  const int ti = xi % ctas_per_block;
  sl.b = blockIdx.y / L.Hq;
  sl.hq = blockIdx.y % L.Hq;
  sl.hkv = sl.hq / (L.Hq / L.Hkv);
  sl.q0 = (long long)j * C + (long long)ti * (BM * NQ);
  const long long q_blk_end = min(T, (long long)(j + 1) * C);
  if (sl.q0 >= q_blk_end) return;
  if ((tc::smem_u32(smem) & 1023u) != 0) {  // operand tiles need 1024-byte alignment
    if (tid == 0) atomicExch(status, KVM_ERR_UNSUPPORTED);
    return;
  }
  // what does not depend on the plan: window start, window tiles per query tile, leading window tiles
  sl.bb = max(0LL, (long long)(j + 1 - L.W) * C);
  sl.lead = kLeadWindowTiles;
  int nw[NQ];
#pragma unroll
  for (int qi = 0; qi < NQ; ++qi) {
    const long long qs = sl.q0 + (long long)qi * BM;
    sl.q_end[qi] = min(q_blk_end, qs + BM);
    nw[qi] = qs < q_blk_end ? (int)((sl.q_end[qi] - sl.bb + BN - 1) / BN) : 0;
    if (qs < q_blk_end) sl.lead = min(sl.lead, nw[qi]);
  }
  sl.q_end_all = min(q_blk_end, sl.q0 + (long long)BM * NQ);

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&bars->q_full[i], 1);
      tc::mbar_init(&bars->s_full[i][0], 1);
      tc::mbar_init(&bars->s_full[i][1], 1);
      tc::mbar_init(&bars->p_full[i][0], 4);
      tc::mbar_init(&bars->p_full[i][1], 4);
      tc::mbar_init(&bars->pv_done[i], 1);
      tc::mbar_init(&bars->o_final[i], 1);
      tc::mbar_init(&bars->o_ready[i], 4);
    }
    for (int i = 0; i < kStages; ++i) {
      tc::mbar_init(&bars->kv_full[i], 1);
      tc::mbar_init(&bars->kv_empty[i], NQ);
    }
    tc::fence_barrier_init();
    // the copies that need nothing from the plan start now; the plan entry is read behind them
#pragma unroll
    for (int qi = 0; qi < NQ; ++qi)
      if (nw[qi] > 0) issue_query_tile<NQ>(smem, bars, &maps, sl.b, sl.hq, qi, (int)(sl.q0 + (long long)qi * BM));
    for (int t = 0; t < sl.lead; ++t)
      issue_window_tile<NQ>(smem, bars, &maps, sl.b, sl.hkv, t, (int)(sl.bb + (long long)t * BN));
  }
  if (warp == CF::kMmaWarp) tc::tmem_alloc(&bars->tmem_base, CF::kTmemCols);
  sl.S = 0;
  sl.mk = sl.mv = nullptr;
  sl.midx = nullptr;
  if (j >= L.W) {
    const kvm_update_plan pl = plan[j - L.W];
    sl.S = pl.state_before + pl.n_append;
    const size_t kvrow = (size_t)(sl.b * L.Hkv + sl.hkv);
    sl.mk = pool_k + kvrow * pool_rows * HD;
    sl.mv = pool_v + kvrow * pool_rows * HD;
    sl.midx = ver_idx + kvrow * ver_rows + pl.version_row;
  }
  sl.n_mem_tiles = (sl.S + BN - 1) / BN;
  sl.n_max = 0;
#pragma unroll
  for (int qi = 0; qi < NQ; ++qi) {
    sl.n_tiles[qi] = nw[qi] > 0 ? sl.n_mem_tiles + nw[qi] : 0;
    sl.n_max = max(sl.n_max, sl.n_tiles[qi]);
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;

  bool ok = true;
  if (warp < CF::kSoftmaxWarps) {
    ok = softmax_role<NQ>(sl, L, smem, bars, tmem, warp >> 2, tid & 127, warp & 3, lane, sm_scale, &maps);
  } else if (warp < CF::kMmaWarp) {
    ok = loader_role<NQ>(sl, smem, bars, warp - CF::kSoftmaxWarps, lane, &maps);
    cp_async_wait<0>();
  } else {
    if (lane == 0) ok = mma_role<NQ>(sl, smem, bars, tmem, warp - CF::kMmaWarp);
    __syncwarp();
  }
  if (!ok) atomicExch(status, KVM_ERR_DEVICE_TIMEOUT);
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == CF::kMmaWarp) tc::tmem_dealloc(tmem, CF::kTmemCols);
}

template <int NQ>
static cudaError_t launch_nq(const LayerDev& L, int batch, long long T, Tensor4 q, Tensor4 k, Tensor4 v,
                             const kvm_update_plan* plan_dev, const bf16* pool_k, const bf16* pool_v, long long pool_rows,
                             const int* ver_idx, long long ver_rows, bf16* out, int* status, cudaStream_t stream,
                             const GatherDst* gd) {
  using CF = Cfg<NQ>;
  const int n_qblocks = (int)((T + L.C - 1) / L.C);
  const int ctas_per_block = L.C / (BM * NQ);
  cudaError_t e = cudaFuncSetAttribute(kvm_attn_prefill_tc_kernel<NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)CF::kSmemBytes);
  if (e != cudaSuccess) return e;
  AttnMaps maps;
  // dimensions ordered by stride: [B,T,H,D] storage (heads inside tokens) or [B,H,T,D] storage
  auto encode = [&](CUtensorMap* m, const Tensor4& t, int heads, int box_rows, bool head_inner) {
    if (head_inner) {
      const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)heads, (cuuint64_t)T, (cuuint64_t)batch};
      const cuuint64_t strides[3] = {(cuuint64_t)t.sh * 2, (cuuint64_t)t.st * 2, (cuuint64_t)t.sb * 2};
      const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
      return encode_bf16_map(m, t.ptr, 4, dims, strides, box);
    }
    const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)T, (cuuint64_t)heads, (cuuint64_t)batch};
    const cuuint64_t strides[3] = {(cuuint64_t)t.st * 2, (cuuint64_t)t.sh * 2, (cuuint64_t)t.sb * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
    return encode_bf16_map(m, t.ptr, 4, dims, strides, box);
  };
  maps.q_head_inner = q.sh < q.st ? 1 : 0;
  maps.kv_head_inner = k.sh < k.st ? 1 : 0;
  if ((v.sh < v.st) != (k.sh < k.st)) return cudaErrorInvalidValue;  // keys and values share one layout
  const int out_heads = gd ? L.Hq * gd->n_ranks : L.Hq;
  Tensor4 o4;  // the output [B, T, heads*D] seen as [batch][head][token][D]
  o4.ptr = gd ? static_cast<const bf16*>(gd->base[gd->rank]) : out;
  o4.sb = T * (long long)out_heads * HD;
  o4.st = (long long)out_heads * HD;
  o4.sh = HD;
  if (!encode(&maps.q, q, L.Hq, BM, maps.q_head_inner != 0) || !encode(&maps.k, k, L.Hkv, BN, maps.kv_head_inner != 0) ||
      !encode(&maps.v, v, L.Hkv, BN, maps.kv_head_inner != 0) || !encode(&maps.o, o4, out_heads, BM, true))
    return cudaErrorInvalidValue;
  maps.n_peer = 0;
  maps.h_off = gd ? gd->rank * L.Hq : 0;
  if (gd) {
    for (int r = 0; r < gd->n_ranks; ++r) {
      if (r == gd->rank) continue;
      o4.ptr = static_cast<const bf16*>(gd->base[r]);
      if (!encode(&maps.o_peer[maps.n_peer++], o4, out_heads, BM, true)) return cudaErrorInvalidValue;
    }
  }
  dim3 grid(n_qblocks * ctas_per_block, batch * L.Hq);
  kvm_attn_prefill_tc_kernel<NQ><<<grid, CF::kThreads, CF::kSmemBytes, stream>>>(
      L, T, q, k, v, plan_dev, pool_k, pool_v, pool_rows, ver_idx, ver_rows, out, ctas_per_block,
      1.0f / sqrtf((float)HD), status, maps);
  return cudaGetLastError();
}


cudaError_t launch_attn_tc(const LayerDev& L, int batch, long long T, Tensor4 q, Tensor4 k, Tensor4 v,
                           const kvm_update_plan* plan_dev, const bf16* pool_k, const bf16* pool_v, long long pool_rows,
                           const int* ver_idx, long long ver_rows, bf16* out, int* status, cudaStream_t stream,
                           const GatherDst* gd) {
  if (gd && (gd->n_ranks < 2 || gd->n_ranks > 8 || gd->rank < 0 || gd->rank >= gd->n_ranks)) return cudaErrorInvalidValue;
  if (L.C % 256 == 0)
    return launch_nq<2>(L, batch, T, q, k, v, plan_dev, pool_k, pool_v, pool_rows, ver_idx, ver_rows, out, status, stream, gd);
  return launch_nq<1>(L, batch, T, q, k, v, plan_dev, pool_k, pool_v, pool_rows, ver_idx, ver_rows, out, status, stream, gd);
}

}  // namespace kvm
