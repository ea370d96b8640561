// Block-recurrent memory update of one kv row, executed by one thread block.
//
// Follows the reference's eager update (model/kvm_mixer.py:250-340) with the fp32 merge routing of
// model/kvm_fp32_routing_reference.py:24-49:
//   1. prepared keys pk = LN(zero-rope(k)), gated streams gk = bf16(pk*g), gv = bf16(v*g)
//   2. novelty score of every token = max over the OLD memory of bf16(pk . k_attn)   (tensor cores)
//      the n_append lowest scores (stable by token index) are appended, in token order
//   3. merge routing: argmax over the memory AFTER the appends of the fp32 logits gk . k_attn
//      (tensor cores, fp32 accumulate), leading `sink` rows excluded, lowest index wins ties
//   4. per touched row: delta = sum of the routed gk (gv) rows in token order (fp32),
//      row = bf16(row + bf16(delta)), then the attention view of the row is recomputed.
// The order of every floating-point sum is fixed, so two runs give identical bits.
#pragma once

#include "kvm_common.cuh"

namespace kvm {

constexpr int kScanTile = 64;  // memory rows per shared-memory tile of the routing GEMM

struct TokenSrc {  // the C tokens consumed by one update; token t at base + t*stride
  const bf16* k;
  long long k_st;
  const bf16* v;
  long long v_st;
  const bf16* g;
  long long g_st;
};

struct MemoryRowPtrs {  // the memory of one kv row
  bf16* k_sum;
  bf16* v_sum;
  float* vlen;
  bf16* k_attn;
  bf16* v_attn;
};

template <int D>
__host__ __device__ constexpr int scan_tile_stride() { return D + 8; }

// Shared-memory carve-up of the update (sizes depend on C and on the memory capacity).
template <int D>
struct UpdateSmem {
  bf16* btile;   // [2][kScanTile][D+8]
  float* app;    // [C] novelty score
  float* best;   // [C] best merge logit
  int* idx;      // [C] best merge row, later: route (row >= 0 merged, -(1+row) appended)
  int* pos;      // [C] position inside the append list / inside the routed row's token list
  int* flag;     // [C] 1 = appended
  int* list;     // [C] merged tokens grouped by row, token order inside a group
  int* touched;  // [C] rows that received at least one token
  int* cnt;      // [capacity]
  int* start;    // [capacity]
  int* counters; // [4]
  __host__ __device__ static size_t bytes(int C, int capacity) {
    size_t b = (size_t)2 * kScanTile * scan_tile_stride<D>() * sizeof(bf16);
    b += (size_t)C * 4 * 7;
    b += (size_t)capacity * 4 * 2;
    b += 16;
    return b;
  }
  __device__ void carve(unsigned char* base, int C, int capacity) {
    btile = reinterpret_cast<bf16*>(base);
    base += (size_t)2 * kScanTile * scan_tile_stride<D>() * sizeof(bf16);
    app = reinterpret_cast<float*>(base); base += (size_t)C * 4;
    best = reinterpret_cast<float*>(base); base += (size_t)C * 4;
    idx = reinterpret_cast<int*>(base); base += (size_t)C * 4;
    pos = reinterpret_cast<int*>(base); base += (size_t)C * 4;
    flag = reinterpret_cast<int*>(base); base += (size_t)C * 4;
    list = reinterpret_cast<int*>(base); base += (size_t)C * 4;
    touched = reinterpret_cast<int*>(base); base += (size_t)C * 4;
    cnt = reinterpret_cast<int*>(base); base += (size_t)capacity * 4;
    start = reinterpret_cast<int*>(base); base += (size_t)capacity * 4;
    counters = reinterpret_cast<int*>(base);
  }
};

// Issue the cp.async copies of one tile of memory rows [row0, row0+kScanTile) (rows >= n_end zero-filled).
template <int D, int NT>
__device__ __forceinline__ void scan_load_tile(bf16* dst, const bf16* k_attn, int row0, int n_end, int tid) {
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  constexpr int STR = scan_tile_stride<D>();
  for (int c = tid; c < kScanTile * CPR; c += NT) {
    int r = c / CPR, cc = c % CPR;
    int row = row0 + r;
    bool ok = row < n_end;
    const bf16* src = k_attn + (size_t)(ok ? row : 0) * D + cc * 8;
    cp_async16(dst + r * STR + cc * 8, src, ok ? 16 : 0);
  }
}

// Routing GEMM over memory rows [n_begin, n_end): per token the running maximum of the bf16-rounded
// pk scores (novelty, only if want_app) and the running fp32 argmax of the gk logits (rows below
// `protected_rows` excluded).  Results are merged into s.app / s.best / s.idx.
template <int D, int NT>
__device__ void scan_memory(const bf16* __restrict__ pk, const bf16* __restrict__ gk, int C,
                            const bf16* __restrict__ k_attn, int n_begin, int n_end, bool want_app,
                            int protected_rows, UpdateSmem<D>& s) {
  constexpr int NW = NT / 32;
  constexpr int KS = D / 16;
  constexpr int STR = scan_tile_stride<D>();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_mtiles = C / 16;
  const int n_tiles = (n_end - n_begin + kScanTile - 1) / kScanTile;
  if (n_tiles <= 0) return;

  for (int pass0 = 0; pass0 < n_mtiles; pass0 += NW) {
    const int mt = pass0 + warp;
    const bool active = mt < n_mtiles;
    uint32_t ap[KS][4], ag[KS][4];
    if (active) {
      const int r0 = mt * 16 + g, r1 = r0 + 8;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int c0 = ks * 16 + t * 2;
        ag[ks][0] = *reinterpret_cast<const uint32_t*>(gk + (size_t)r0 * D + c0);
        ag[ks][1] = *reinterpret_cast<const uint32_t*>(gk + (size_t)r1 * D + c0);
        ag[ks][2] = *reinterpret_cast<const uint32_t*>(gk + (size_t)r0 * D + c0 + 8);
        ag[ks][3] = *reinterpret_cast<const uint32_t*>(gk + (size_t)r1 * D + c0 + 8);
        if (want_app) {
          ap[ks][0] = *reinterpret_cast<const uint32_t*>(pk + (size_t)r0 * D + c0);
          ap[ks][1] = *reinterpret_cast<const uint32_t*>(pk + (size_t)r1 * D + c0);
          ap[ks][2] = *reinterpret_cast<const uint32_t*>(pk + (size_t)r0 * D + c0 + 8);
          ap[ks][3] = *reinterpret_cast<const uint32_t*>(pk + (size_t)r1 * D + c0 + 8);
        } else {
          ap[ks][0] = ap[ks][1] = ap[ks][2] = ap[ks][3] = 0u;
        }
      }
    }
    float amax[2] = {-INFINITY, -INFINITY};
    float bbest[2] = {-INFINITY, -INFINITY};
    int bidx[2] = {-1, -1};

    __syncthreads();  // previous users of the tile buffers are done
    scan_load_tile<D, NT>(s.btile, k_attn, n_begin, n_end, tid);
    cp_async_commit();
    for (int it = 0; it < n_tiles; ++it) {
      const int cur = it & 1;
      if (it + 1 < n_tiles) {
        scan_load_tile<D, NT>(s.btile + (size_t)(cur ^ 1) * kScanTile * STR, k_attn,
                              n_begin + (it + 1) * kScanTile, n_end, tid);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      if (active) {
        const bf16* bt = s.btile + (size_t)cur * kScanTile * STR;
        const int tile_base = n_begin + it * kScanTile;
#pragma unroll
        for (int nt = 0; nt < kScanTile / 8; ++nt) {
          if (tile_base + nt * 8 >= n_end) break;
          float cg[4] = {0.f, 0.f, 0.f, 0.f}, cp[4] = {0.f, 0.f, 0.f, 0.f};
          const bf16* brow = bt + (size_t)(nt * 8 + g) * STR + t * 2;
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + ks * 16);
            uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + ks * 16 + 8);
            mma_bf16_16816(cg, ag[ks], b0, b1);
            if (want_app) mma_bf16_16816(cp, ap[ks], b0, b1);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const int n = tile_base + nt * 8 + t * 2 + (e & 1);
            if (n < n_end) {
              if (want_app) amax[r] = fmaxf(amax[r], bf16_round(cp[e]));
              if (n >= protected_rows && (cg[e] > bbest[r] || bidx[r] < 0)) {
                bbest[r] = cg[e];
                bidx[r] = n;
              }
            }
          }
        }
      }
      __syncthreads();  // tile `cur` may be overwritten by the next prefetch
    }
    if (active) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
#pragma unroll
        for (int off = 1; off <= 2; off <<= 1) {
          float ob = __shfl_xor_sync(0xffffffffu, bbest[r], off);
          int oi = __shfl_xor_sync(0xffffffffu, bidx[r], off);
          float oa = __shfl_xor_sync(0xffffffffu, amax[r], off);
          amax[r] = fmaxf(amax[r], oa);
          if (oi >= 0 && (bidx[r] < 0 || ob > bbest[r] || (ob == bbest[r] && oi < bidx[r]))) {
            bbest[r] = ob;
            bidx[r] = oi;
          }
        }
        if (t == 0) {
          const int row = mt * 16 + g + r * 8;
          if (want_app) s.app[row] = amax[r];
          if (bidx[r] >= 0 && (s.idx[row] < 0 || bbest[r] > s.best[row])) {
            s.best[row] = bbest[r];
            s.idx[row] = bidx[r];
          }
        }
      }
    }
  }
  __syncthreads();
}

// One full update of one kv row.  `pk_scr` / `gk_scr` are [C][D] bf16 global scratch rows private to
// this block.  `route_out` ([C] int32, may be null) receives the decision for every token.
template <int D, int NT>
__device__ void memory_update(const LayerDev& L, const TokenSrc& src, const MemoryRowPtrs& mem, int capacity,
                              int S_before, int n_append, bf16* pk_scr, bf16* gk_scr, int* route_out,
                              UpdateSmem<D>& s) {
  constexpr int NW = NT / 32;
  const int C = L.C;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S_after = S_before + n_append;
  const int n_merge = C - n_append;

  // ---- 1. prepared / gated keys of the block -> scratch
  for (int tkn = warp; tkn < C; tkn += NW) {
    RowVec<D> r;
    prepare_key_row<D>(L, r, src.k + (long long)tkn * src.k_st, lane);
    store_row<D>(r, pk_scr + (size_t)tkn * D, lane);
    if (L.gate_keys) {
      const float gt = __bfloat162float(src.g[(long long)tkn * src.g_st]);
#pragma unroll
      for (int i = 0; i < D / 32; ++i) r.x[i] = bf16_round(r.x[i] * gt);
    }
    store_row<D>(r, gk_scr + (size_t)tkn * D, lane);
  }
  for (int i = tid; i < C; i += NT) {
    s.app[i] = -INFINITY;
    s.best[i] = -INFINITY;
    s.idx[i] = -1;
    s.pos[i] = 0;
    s.flag[i] = (n_merge == 0) ? 1 : 0;
  }
  if (tid < 4) s.counters[tid] = 0;
  __syncthreads();

  const int protected_rows = min(L.sink_len, S_after);

  // ---- 2. scores against the old memory, append selection
  if (n_merge > 0) scan_memory<D, NT>(pk_scr, gk_scr, C, mem.k_attn, 0, S_before, n_append > 0, protected_rows, s);
  if (n_append > 0 && n_merge > 0) {
    for (int i = tid; i < C; i += NT) {
      const float si = s.app[i];
      int rank = 0;
      for (int u = 0; u < C; ++u) {
        const float su = s.app[u];
        rank += (su < si || (su == si && u < i)) ? 1 : 0;
      }
      s.flag[i] = rank < n_append ? 1 : 0;
    }
    __syncthreads();
  }
  if (n_append > 0) {
    for (int i = tid; i < C; i += NT) {
      int p = 0;
      for (int u = 0; u < i; ++u) p += s.flag[u];
      s.pos[i] = p;
    }
    __syncthreads();
    // appended rows, in token order
    for (int tkn = warp; tkn < C; tkn += NW) {
      if (!s.flag[tkn]) continue;
      const int row = S_before + s.pos[tkn];
      if (row >= capacity) continue;  // guarded by the host-side capacity check
      RowVec<D> kr, vr;
      load_row<D>(kr, (L.gate_appends ? gk_scr : pk_scr) + (size_t)tkn * D, lane);
      load_row<D>(vr, src.v + (long long)tkn * src.v_st, lane);
      if (L.gate_appends && L.gate_values) {
        const float gt = __bfloat162float(src.g[(long long)tkn * src.g_st]);
#pragma unroll
        for (int i = 0; i < D / 32; ++i) vr.x[i] = bf16_round(vr.x[i] * gt);
      }
      const float vl = row_norm<D>(vr);
      store_row<D>(kr, mem.k_sum + (size_t)row * D, lane);
      store_row<D>(vr, mem.v_sum + (size_t)row * D, lane);
      if (lane == 0) mem.vlen[row] = vl;
      refresh_memory_row<D>(L, kr, vr, vl, mem.k_attn + (size_t)row * D, mem.v_attn + (size_t)row * D, lane);
    }
    __syncthreads();
  }
  if (n_merge == 0) {
    if (route_out)
      for (int i = tid; i < C; i += NT) route_out[i] = -(1 + S_before + s.pos[i]);
    __syncthreads();
    return;
  }

  // ---- 3. merge targets among the rows that were just appended (append-before-merge)
  if (n_append > 0) scan_memory<D, NT>(pk_scr, gk_scr, C, mem.k_attn, S_before, S_after, false, protected_rows, s);

  // ---- 4. group the merged tokens by target row, token order inside a group
  for (int i = tid; i < S_after; i += NT) s.cnt[i] = 0;
  __syncthreads();
  if (warp == 0) {
    for (int base = 0; base < C; base += 32) {
      const int tkn = base + lane;
      const bool merged = tkn < C && !s.flag[tkn] && s.idx[tkn] >= 0;
      const int row = merged ? s.idx[tkn] : -(1 + lane);
      const unsigned grp = __match_any_sync(0xffffffffu, row);
      if (merged) {
        s.pos[tkn] = s.cnt[row] + __popc(grp & ((1u << lane) - 1u));
      }
      __syncwarp();
      if (merged && (int)(__ffs(grp) - 1) == lane) s.cnt[row] += __popc(grp);
      __syncwarp();
    }
  }
  __syncthreads();
  for (int i = tid; i < C; i += NT) {
    if (!s.flag[i] && s.idx[i] >= 0 && s.pos[i] == 0) {
      const int row = s.idx[i];
      s.start[row] = atomicAdd(&s.counters[0], s.cnt[row]);
      s.touched[atomicAdd(&s.counters[1], 1)] = row;
    }
  }
  __syncthreads();
  for (int i = tid; i < C; i += NT) {
    if (!s.flag[i] && s.idx[i] >= 0) s.list[s.start[s.idx[i]] + s.pos[i]] = i;
    if (route_out) route_out[i] = s.flag[i] ? -(1 + S_before + s.pos[i]) : s.idx[i];
  }
  __syncthreads();

  // ---- 5. fixed-order accumulation into the touched rows and refresh of their attention view
  const int n_touched = s.counters[1];
  for (int i = warp; i < n_touched; i += NW) {
    const int row = s.touched[i];
    const int n = s.cnt[row];
    const int b0 = s.start[row];
    RowVec<D> ak, av;
#pragma unroll
    for (int e = 0; e < D / 32; ++e) ak.x[e] = av.x[e] = 0.f;
    for (int j = 0; j < n; ++j) {
      const int tkn = s.list[b0 + j];
      RowVec<D> kr, vr;
      load_row<D>(kr, gk_scr + (size_t)tkn * D, lane);
      load_row<D>(vr, src.v + (long long)tkn * src.v_st, lane);
      if (L.gate_values) {
        const float gt = __bfloat162float(src.g[(long long)tkn * src.g_st]);
#pragma unroll
        for (int e = 0; e < D / 32; ++e) vr.x[e] = bf16_round(vr.x[e] * gt);
      }
#pragma unroll
      for (int e = 0; e < D / 32; ++e) {
        ak.x[e] += kr.x[e];
        av.x[e] += vr.x[e];
      }
    }
    RowVec<D> ks, vs;
    load_row<D>(ks, mem.k_sum + (size_t)row * D, lane);
    load_row<D>(vs, mem.v_sum + (size_t)row * D, lane);
#pragma unroll
    for (int e = 0; e < D / 32; ++e) {
      ks.x[e] = bf16_round(ks.x[e] + bf16_round(ak.x[e]));
      vs.x[e] = bf16_round(vs.x[e] + bf16_round(av.x[e]));
    }
    store_row<D>(ks, mem.k_sum + (size_t)row * D, lane);
    store_row<D>(vs, mem.v_sum + (size_t)row * D, lane);
    refresh_memory_row<D>(L, ks, vs, mem.vlen[row], mem.k_attn + (size_t)row * D, mem.v_attn + (size_t)row * D, lane);
  }
  __syncthreads();
}

}  // namespace kvm
