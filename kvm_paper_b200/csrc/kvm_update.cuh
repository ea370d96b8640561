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
//
// The update sits on a strictly sequential chain (one update per block and kv row), so it is organised
// for latency: when it fits (SB = true) the whole token block -- keys, values, gates -- is pulled into
// shared memory with one wave of cp.async and every later phase works from there; only the prepared
// key is kept (the gated key is re-derived on the fly, the product of two bf16 numbers rounds the same
// way everywhere).
#pragma once

#include "kvm_common.cuh"
#include "kvm_tc.cuh"

namespace kvm {

constexpr int kScanTile = 64;  // memory rows per shared-memory tile of the routing GEMM
constexpr int kMaxCluster = 4; // CTAs that may share one kv row
constexpr int kDirectRows = 4; // up to this many appended rows are scored with plain dot products

struct TokenSrc {  // the C tokens consumed by one update; token t at base + t*stride
  const bf16* k;
  long long k_st;
  const bf16* v;
  long long v_st;
  const bf16* g;
  long long g_st;
  const bf16* next_k;  // first row of the block the NEXT update consumes (L2 prefetch), or null
  const bf16* next_v;
};

struct MemoryRowPtrs {  // the memory of one kv row
  bf16* k_sum;
  bf16* v_sum;
  float* vlen;
  bf16* k_attn;
  bf16* v_attn;
};

struct BlockView {  // where the phases after the load find the block's data
  const bf16* pk;   // prepared keys, row stride pk_st elements ...
  int pk_st;
  int swz_rows;     // ... or, if non-zero (D = 128): two blocks of [swz_rows][64 elements] in the 128-byte swizzle
                    // (16-byte piece c of row r at position c ^ (r % 8)), the tcgen05 operand layout
  // 16-byte piece c (elements 8c .. 8c+7) of row r
  __device__ __forceinline__ const bf16* pk_piece(int r, int c) const {
    if (swz_rows)
      return reinterpret_cast<const bf16*>(reinterpret_cast<const unsigned char*>(pk) + (size_t)(c >> 3) * swz_rows * 128 +
                                           r * 128 + (((c & 7) ^ (r & 7)) << 4));
    return pk + (size_t)r * pk_st + c * 8;
  }
  const bf16* v;    // values, row stride v_st elements
  long long v_st;
  const float* g;   // gates [C] (shared memory)
};

template <int D>
__host__ __device__ constexpr int scan_tile_stride() { return D + 8; }

// Shared-memory carve-up of the update (sizes depend on C, the memory capacity and SB).
template <int D>
struct UpdateSmem {
  bf16* btile;   // [2][kScanTile][D+8]
  bf16* pk_s;    // [C][D+8]   (SB only)
  bf16* v_s;     // [C][D]     (SB only)
  float* g_s;    // [C] gates
  float* app;    // [C] novelty score
  float* best;   // [C] best merge logit
  int* idx;      // [C] merge target row (-1 for appended tokens once grouping starts)
  int* pos;      // [C] position inside the append list
  int* flag;     // [C] 1 = appended
  int* ord;      // [C] position of a merged token inside its target row's token list
  int* lead;     // [C] first token routed to the same row
  int* tcnt;     // [C] (by leading token) tokens routed to the row
  int* tstart;   // [C] (by leading token) start of the row's token list inside `list`
  int* list;     // [C] merged tokens grouped by row, token order inside a group
  int* touched;  // [C] leading tokens, one per row that received tokens
  int* cur;      // [capacity] pool slot holding the attention view of each memory row (pool mode)
  int* counters; // [4 + 32]
  float* xapp;   // [kMaxCluster][C] partial novelty maxima of the CTAs of a cluster
  float* xbest;  // [kMaxCluster][C] partial best logits
  int* xidx;     // [kMaxCluster][C] partial best rows
  uint64_t* bars;  // [2] mbarriers of the tcgen05 routing scan, [2] = slot for the tensor-memory base address
  uint32_t tmem;   // tensor-memory base (valid when use_tc)
  bool use_tc;     // the tcgen05 routing scan is available (tensor memory allocated, barriers initialised once)
  uint32_t tc_tiles;  // tiles issued so far by the tcgen05 scan: tile n signals barrier n%2 with phase parity (n/2)%2
  int* status;     // device status word (a bounded wait that ran out is reported here), or null
  static constexpr int kTokenArrays = 13 + 3 * kMaxCluster;
  __host__ __device__ static size_t bytes(int C, int capacity, bool sb) {
    size_t b = (size_t)2 * kScanTile * scan_tile_stride<D>() * sizeof(bf16);
    if (sb) b += (size_t)C * (D + 8) * sizeof(bf16) + (size_t)C * D * sizeof(bf16);
    b += (size_t)C * 4 * kTokenArrays;
    b += (size_t)((capacity + 3) / 4 * 4) * 4;
    b += 36 * 4 + 32;
    return b;
  }
  __device__ void carve(unsigned char* base, int C, int capacity, bool sb) {
    btile = reinterpret_cast<bf16*>(base);
    base += (size_t)2 * kScanTile * scan_tile_stride<D>() * sizeof(bf16);
    pk_s = v_s = nullptr;
    if (sb) {
      pk_s = reinterpret_cast<bf16*>(base); base += (size_t)C * (D + 8) * sizeof(bf16);
      v_s = reinterpret_cast<bf16*>(base); base += (size_t)C * D * sizeof(bf16);
    }
    int** arr[13] = {reinterpret_cast<int**>(&g_s), reinterpret_cast<int**>(&app), reinterpret_cast<int**>(&best),
                               &idx, &pos, &flag, &ord, &lead, &tcnt, &tstart, &list, &touched, nullptr};
    for (int i = 0; i < 12; ++i) {
      *arr[i] = reinterpret_cast<int*>(base);
      base += (size_t)C * 4;
    }
    base += (size_t)C * 4;  // spare
    xapp = reinterpret_cast<float*>(base); base += (size_t)kMaxCluster * C * 4;
    xbest = reinterpret_cast<float*>(base); base += (size_t)kMaxCluster * C * 4;
    xidx = reinterpret_cast<int*>(base); base += (size_t)kMaxCluster * C * 4;
    cur = reinterpret_cast<int*>(base); base += (size_t)((capacity + 3) / 4 * 4) * 4;
    counters = reinterpret_cast<int*>(base); base += 36 * 4;
    bars = reinterpret_cast<uint64_t*>(base);
    tmem = 0;
    use_tc = false;
    tc_tiles = 0;
    status = nullptr;
  }
};

constexpr size_t kSmemLimit = 225 * 1024;  // dynamic part: the kernels also hold ~1 KB of static shared memory

template <int D>
__host__ __device__ inline bool update_block_fits_smem(int C, int capacity) {
  return UpdateSmem<D>::bytes(C, capacity, true) <= kSmemLimit;
}

// A cluster of up to kMaxCluster CTAs may share one kv row: the memory rows of the routing scan and the
// touched rows of the scatter are split between them, partial routing results are exchanged through
// distributed shared memory, everything else is computed redundantly (it is deterministic).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_smem_addr(const void* local, int peer) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(local), r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(peer));
  return r;
}
__device__ __forceinline__ void st_peer_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_peer_s32(uint32_t addr, int v) {
  asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, __nv_bfloat162 g2) {
  __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&a);
  x = __hmul2(x, g2);
  return *reinterpret_cast<uint32_t*>(&x);
}

// acc += row (optionally times the gate, rounded to bf16 first) for the EPL elements of this lane; the gated
// product is formed on packed bf16 pairs (the product of two bf16 numbers rounds the same way everywhere).
template <int D, int GL>
__device__ __forceinline__ void accumulate_row(RowVec<D, GL>& acc, const bf16* row, int gl, bool gated, float gate) {
  constexpr int EPL = D / GL;
  const bf16* p = row + gl * EPL;
  const __nv_bfloat162 g2 = __float2bfloat162_rn(gate);
  if constexpr (EPL % 8 == 0) {
#pragma unroll
    for (int c = 0; c < EPL / 8; ++c) {
      uint4 u = *reinterpret_cast<const uint4*>(p + c * 8);
      if (gated) {
        u.x = mul_bf16x2(u.x, g2);
        u.y = mul_bf16x2(u.y, g2);
        u.z = mul_bf16x2(u.z, g2);
        u.w = mul_bf16x2(u.w, g2);
      }
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), d = unpack_bf16(u.z), e = unpack_bf16(u.w);
      acc.x[c * 8 + 0] += a.x; acc.x[c * 8 + 1] += a.y; acc.x[c * 8 + 2] += b.x; acc.x[c * 8 + 3] += b.y;
      acc.x[c * 8 + 4] += d.x; acc.x[c * 8 + 5] += d.y; acc.x[c * 8 + 6] += e.x; acc.x[c * 8 + 7] += e.y;
    }
  } else {
    RowVec<D, GL> r;
    load_row<D, GL>(r, row, gl);
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc.x[e] += gated ? bf16_round(r.x[e] * gate) : r.x[e];
  }
}

// The EPL elements of this lane of prepared-key row `row` (either layout of the block view).
template <int D, int GL>
__device__ __forceinline__ void load_pk_row(RowVec<D, GL>& r, const BlockView& blk, int row, int gl) {
  constexpr int EPL = D / GL;
  if constexpr (EPL % 8 == 0) {
#pragma unroll
    for (int c = 0; c < EPL / 8; ++c) {
      const uint4 u = *reinterpret_cast<const uint4*>(blk.pk_piece(row, gl * (EPL / 8) + c));
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), d = unpack_bf16(u.z), e = unpack_bf16(u.w);
      r.x[c * 8 + 0] = a.x; r.x[c * 8 + 1] = a.y; r.x[c * 8 + 2] = b.x; r.x[c * 8 + 3] = b.y;
      r.x[c * 8 + 4] = d.x; r.x[c * 8 + 5] = d.y; r.x[c * 8 + 6] = e.x; r.x[c * 8 + 7] = e.y;
    }
  } else {
    load_row<D, GL>(r, blk.pk + (size_t)row * blk.pk_st, gl);
  }
}
// accumulate_row for a prepared-key row of the block view
template <int D, int GL>
__device__ __forceinline__ void accumulate_pk_row(RowVec<D, GL>& acc, const BlockView& blk, int row, int gl, bool gated, float gate) {
  constexpr int EPL = D / GL;
  if constexpr (EPL % 8 == 0) {
    const __nv_bfloat162 g2 = __float2bfloat162_rn(gate);
#pragma unroll
    for (int c = 0; c < EPL / 8; ++c) {
      uint4 u = *reinterpret_cast<const uint4*>(blk.pk_piece(row, gl * (EPL / 8) + c));
      if (gated) {
        u.x = mul_bf16x2(u.x, g2);
        u.y = mul_bf16x2(u.y, g2);
        u.z = mul_bf16x2(u.z, g2);
        u.w = mul_bf16x2(u.w, g2);
      }
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), d = unpack_bf16(u.z), e = unpack_bf16(u.w);
      acc.x[c * 8 + 0] += a.x; acc.x[c * 8 + 1] += a.y; acc.x[c * 8 + 2] += b.x; acc.x[c * 8 + 3] += b.y;
      acc.x[c * 8 + 4] += d.x; acc.x[c * 8 + 5] += d.y; acc.x[c * 8 + 6] += e.x; acc.x[c * 8 + 7] += e.y;
    }
  } else {
    accumulate_row<D, GL>(acc, blk.pk + (size_t)row * blk.pk_st, gl, gated, gate);
  }
}

// Issue the cp.async copies of one tile of memory rows [row0, row0+kScanTile) (rows >= n_end zero-filled).
// `slots` (shared memory, may be null = identity) maps a memory row to the row of `k_attn` that holds it.
template <int D, int NT>
__device__ __forceinline__ void scan_load_tile(bf16* dst, const bf16* k_attn, const int* slots, int row0, int n_end, int tid) {
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  constexpr int STR = scan_tile_stride<D>();
  for (int c = tid; c < kScanTile * CPR; c += NT) {
    int r = c / CPR, cc = c % CPR;
    int row = row0 + r;
    bool ok = row < n_end;
    int slot = ok ? (slots ? slots[row] : row) : 0;
    const bf16* src = k_attn + (size_t)slot * D + cc * 8;
    cp_async16(dst + r * STR + cc * 8, src, ok ? 16 : 0);
  }
}

// Routing GEMM over memory rows [n_begin, n_end): per token the running maximum of the bf16-rounded
// pk scores (novelty, only if want_app) and the running fp32 argmax of the gk logits (rows below
// `protected_rows` excluded).  Results are merged into s.app / s.best / s.idx.
template <int D, int NT>
__device__ __noinline__ void scan_memory(const BlockView& blk, bool gate_keys, int C, const bf16* __restrict__ k_attn, const int* slots,
                            int n_begin, int n_end, bool want_app, int protected_rows, UpdateSmem<D>& s) {
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
      const __nv_bfloat162 g0 = __float2bfloat162_rn(blk.g[r0]);
      const __nv_bfloat162 g1 = __float2bfloat162_rn(blk.g[r1]);
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        ap[ks][0] = *reinterpret_cast<const uint32_t*>(blk.pk_piece(r0, ks * 2) + t * 2);
        ap[ks][1] = *reinterpret_cast<const uint32_t*>(blk.pk_piece(r1, ks * 2) + t * 2);
        ap[ks][2] = *reinterpret_cast<const uint32_t*>(blk.pk_piece(r0, ks * 2 + 1) + t * 2);
        ap[ks][3] = *reinterpret_cast<const uint32_t*>(blk.pk_piece(r1, ks * 2 + 1) + t * 2);
        if (gate_keys) {
          ag[ks][0] = mul_bf16x2(ap[ks][0], g0);
          ag[ks][1] = mul_bf16x2(ap[ks][1], g1);
          ag[ks][2] = mul_bf16x2(ap[ks][2], g0);
          ag[ks][3] = mul_bf16x2(ap[ks][3], g1);
        } else {
          ag[ks][0] = ap[ks][0]; ag[ks][1] = ap[ks][1]; ag[ks][2] = ap[ks][2]; ag[ks][3] = ap[ks][3];
        }
      }
    }
    float amax[2] = {-INFINITY, -INFINITY};
    float bbest[2] = {-INFINITY, -INFINITY};
    int bidx[2] = {-1, -1};

    __syncthreads();  // previous users of the tile buffers are done
    scan_load_tile<D, NT>(s.btile, k_attn, slots, n_begin, n_end, tid);
    cp_async_commit();
    for (int it = 0; it < n_tiles; ++it) {
      const int cur = it & 1;
      if (it + 1 < n_tiles) {
        scan_load_tile<D, NT>(s.btile + (size_t)(cur ^ 1) * kScanTile * STR, k_attn, slots,
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
        // two 8-row groups of the tile at a time: four independent accumulation chains keep the MMA pipe fed
#pragma unroll
        for (int nt = 0; nt < kScanTile / 8; nt += 2) {
          if (tile_base + nt * 8 >= n_end) break;
          float cg[2][4], cp[2][4];
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 4; ++e) cg[h][e] = cp[h][e] = 0.f;
          const bf16* brow0 = bt + (size_t)(nt * 8 + g) * STR + t * 2;
          const bf16* brow1 = brow0 + (size_t)8 * STR;
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            const uint32_t b00 = *reinterpret_cast<const uint32_t*>(brow0 + ks * 16);
            const uint32_t b01 = *reinterpret_cast<const uint32_t*>(brow0 + ks * 16 + 8);
            const uint32_t b10 = *reinterpret_cast<const uint32_t*>(brow1 + ks * 16);
            const uint32_t b11 = *reinterpret_cast<const uint32_t*>(brow1 + ks * 16 + 8);
            mma_bf16_16816(cg[0], ag[ks], b00, b01);
            mma_bf16_16816(cg[1], ag[ks], b10, b11);
            if (want_app) {
              mma_bf16_16816(cp[0], ap[ks], b00, b01);
              mma_bf16_16816(cp[1], ap[ks], b10, b11);
            }
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int r = e >> 1;
              const int n = tile_base + (nt + h) * 8 + t * 2 + (e & 1);
              if (n < n_end) {
                if (want_app) amax[r] = fmaxf(amax[r], bf16_round(cp[h][e]));
                if (n >= protected_rows && (cg[h][e] > bbest[r] || bidx[r] < 0)) {
                  bbest[r] = cg[h][e];
                  bidx[r] = n;
                }
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

// ---------------------------------------------------------------------------------------------------
// Routing GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory), for D = 128 and blocks of 128
// or 256 tokens whose prepared keys sit in shared memory in the 128-byte-swizzled K-major operand layout.
// Same contract as scan_memory.  Per tile of 64 memory rows one elected thread issues two groups of MMAs
// (M = 128 tokens each): prepared keys x tile (novelty) and gated keys x tile (merge logits), into one of
// two accumulator buffers in tensor memory; warps 0..7 read back the novelty accumulators (running maximum
// of the bf16-rounded scores), warps 8..15 the merge logits (running fp32 first-argmax), one token row per
// thread and four independent partial results per thread.  The gated keys (A operand of the second group)
// are built once into the shared-memory region that later holds the block's values (fetched after the
// scan) while the first novelty MMAs run.  The first two memory tiles are already in flight when the
// function is entered (`tiles_in_flight`), issued next to the block load.
// Returns false (for every thread) if a bounded wait ran out; nothing has been merged into s.app / s.best /
// s.idx in that case.
constexpr int kTcTile = 64;                       // memory rows per tile of the tcgen05 scan
constexpr uint32_t kTcTmemCols = 512;             // two buffers x (novelty, logits) x two 128-token accumulators x 64

template <int D, int NT>
__device__ __forceinline__ void scan_tc_load_tile(UpdateSmem<D>& s, const bf16* __restrict__ k_attn, const int* slots, int n_begin,
                                                  int n_end, int it) {
  unsigned char* dst = reinterpret_cast<unsigned char*>(s.btile) + (size_t)(it & 1) * (2 * kTcTile * 128);
  const int row0 = n_begin + it * kTcTile;
  for (int c = threadIdx.x; c < kTcTile * 16; c += NT) {
    const int r = c >> 4, cc = c & 15;
    const int row = row0 + r;
    const bool in = row < n_end;
    const int slot = in ? (slots ? slots[row] : row) : 0;
    cp_async16(dst + (cc >> 3) * (kTcTile * 128) + r * 128 + (((cc & 7) ^ (r & 7)) << 4), k_attn + (size_t)slot * D + cc * 8,
               in ? 16 : 0);
  }
}

template <int D, int NT>
__device__ __noinline__ bool scan_memory_tc(const BlockView& blk, bool gate_keys, int C, const bf16* __restrict__ k_attn,
                                            const int* slots, int n_begin, int n_end, bool want_app, int protected_rows,
                                            UpdateSmem<D>& s, int tiles_in_flight) {
  static_assert(D == 128 && NT == 512, "tcgen05 routing scan: head dimension 128, 16 warps");
  constexpr int TN = kTcTile;
  constexpr uint32_t kWaitLimit = 1u << 16;  // the MMAs of one tile take well under a microsecond; ~13 ms before giving up
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = (n_end - n_begin + TN - 1) / TN;
  if (n_tiles <= 0) return true;
  const int n_mt = C / 128;                                              // accumulators of 128 tokens per operand
  const unsigned char* A_pk = reinterpret_cast<const unsigned char*>(blk.pk);   // [2 k-halves][C][128 B], swizzled
  unsigned char* A_gk = reinterpret_cast<unsigned char*>(s.v_s);                 // same layout, gated
  uint64_t* mbar = s.bars;
  constexpr uint32_t idesc = tc::make_idesc(128, TN, 0, 0);
  const uint32_t pk_addr = tc::smem_u32(A_pk), gk_addr = gate_keys ? tc::smem_u32(A_gk) : pk_addr;
  const uint32_t b_addr = tc::smem_u32(s.btile);
  const bool issuer = tid == NT - 32;
  // read-back roles: warps 0..7 novelty (operand 0), warps 8..15 logits (operand 1); warp w -> accumulator (w%8)/4, lanes 32*(w%4)..
  const int op = warp >> 3, mt = (warp >> 2) & 1;
  const bool epi = mt < n_mt && (op == 1 || want_app);
  const uint32_t t_lane = s.tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(op * 128 + mt * TN);
  const uint32_t g0 = s.tc_tiles;  // global index of this call's first tile (barriers are initialised once per kernel)
  bool ok = true;

  // D[buffer it%2][operand][m] += A_operand[m] x tile it
  auto issue_mmas = [&](int it, int operand) {
    const uint32_t a_addr = operand ? gk_addr : pk_addr;
    const uint64_t db0 = tc::make_desc(b_addr + (uint32_t)((it & 1) * (2 * TN * 128)), 16, 1024);
    for (int m = 0; m < n_mt; ++m) {
      const uint64_t da0 = tc::make_desc(a_addr + (uint32_t)(m * 128 * 128), 16, 1024);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint64_t da = da0 + (uint64_t)(((uint32_t)(ks >> 2) * (uint32_t)(C * 128) + (uint32_t)(ks & 3) * 32u) >> 4);
        const uint64_t db = db0 + (uint64_t)(((uint32_t)(ks >> 2) * (uint32_t)(TN * 128) + (uint32_t)(ks & 3) * 32u) >> 4);
        tc::mma_ss(s.tmem + (uint32_t)((it & 1) * 256 + operand * 128 + m * TN), da, db, idesc, ks > 0);
      }
    }
  };
  // four independent running results per thread (columns c % 4), folded at the end: short dependency chains
  float am[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  float bb[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  int bi[4] = {-1, -1, -1, -1};
  auto epilogue = [&](int it) {
    const int tile_base = n_begin + it * TN;
    const int ncols = min(TN, n_end - tile_base);
    const bool full = ncols == TN && tile_base >= protected_rows;  // no column of this tile is masked
    tc::tc_fence_after_sync();
#pragma unroll
    for (int half = 0; half < TN / 32; ++half) {
      if (half * 32 < ncols) {
        uint32_t r[32];
        tc::tmem_ld32(t_lane + (uint32_t)((it & 1) * 256 + half * 32), r);
        tc::tmem_ld_wait();
        const int n0 = tile_base + half * 32;
        if (op == 0) {
          if (full) {
#pragma unroll
            for (int c = 0; c < 32; ++c) am[c & 3] = fmaxf(am[c & 3], bf16_round(__uint_as_float(r[c])));
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c)
              if (n0 + c < n_end) am[c & 3] = fmaxf(am[c & 3], bf16_round(__uint_as_float(r[c])));
          }
        } else {
          if (full) {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const float x = __uint_as_float(r[c]);
              if (x > bb[c & 3] || bi[c & 3] < 0) {
                bb[c & 3] = x;
                bi[c & 3] = n0 + c;
              }
            }
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const float x = __uint_as_float(r[c]);
              const int n = n0 + c;
              if (n < n_end && n >= protected_rows && (x > bb[c & 3] || bi[c & 3] < 0)) {
                bb[c & 3] = x;
                bi[c & 3] = n;
              }
            }
          }
        }
      }
    }
    tc::tc_fence_before_sync();
  };

  // tiles not yet in flight among the first two
  for (int it = tiles_in_flight; it < 2 && it < n_tiles; ++it) scan_tc_load_tile<D, NT>(s, k_attn, slots, n_begin, n_end, it);
  cp_async_commit();
  cp_async_wait<0>();
  tc::fence_proxy_async();
  __syncthreads();  // prepared keys (A operand 0) and the first tiles are in shared memory
  if (issuer && want_app) {  // novelty MMAs of the first tiles run while the gated operand is built
    tc::tc_fence_after_sync();
    for (int it = 0; it < 2 && it < n_tiles; ++it) issue_mmas(it, 0);
  }
  if (gate_keys) {
    // gated keys: the swizzle is a permutation inside 1024-byte groups of 8 rows, so the operand is copied
    // 16-byte unit by unit; unit u of a k-half block belongs to row u / 8
    // (the issuing thread's warp stays out of the copy: its MMAs go out while the others build)
    for (int u = tid; u < C * 16 && warp < NT / 32 - 1; u += NT - 32) {
      const int r = (u & (C * 8 - 1)) >> 3;
      uint4 v = *reinterpret_cast<const uint4*>(A_pk + (size_t)u * 16);
      const __nv_bfloat162 g2 = __float2bfloat162_rn(blk.g[r]);
      v.x = mul_bf16x2(v.x, g2);
      v.y = mul_bf16x2(v.y, g2);
      v.z = mul_bf16x2(v.z, g2);
      v.w = mul_bf16x2(v.w, g2);
      *reinterpret_cast<uint4*>(A_gk + (size_t)u * 16) = v;
    }
    tc::fence_proxy_async();
    __syncthreads();
  }
  if (issuer) {
    tc::tc_fence_after_sync();
    for (int it = 0; it < 2 && it < n_tiles; ++it) {
      issue_mmas(it, 1);
      tc::mma_commit_own_cta(&mbar[(g0 + it) & 1]);  // covers the novelty MMAs of the tile as well (issued earlier)
    }
  }
  for (int it = 0; it < n_tiles; ++it) {
    ok = ok && tc::mbar_wait_limit(&mbar[(g0 + it) & 1], ((g0 + it) >> 1) & 1, kWaitLimit);
    const bool more = it + 2 < n_tiles;
    if (more) {  // the MMAs of tile `it` are done: its operand buffer may be refilled
      scan_tc_load_tile<D, NT>(s, k_attn, slots, n_begin, n_end, it + 2);
      cp_async_commit();
    }
    if (epi) epilogue(it);
    if (more) {
      cp_async_wait<0>();
      tc::fence_proxy_async();
      __syncthreads();  // tile it+2 complete; accumulator buffer it%2 has been read back
      if (issuer) {
        tc::tc_fence_after_sync();
        if (want_app) issue_mmas(it + 2, 0);
        issue_mmas(it + 2, 1);
        tc::mma_commit_own_cta(&mbar[(g0 + it + 2) & 1]);
      }
      }
  }
  s.tc_tiles = g0 + (uint32_t)n_tiles;
  if (!__syncthreads_and(ok ? 1 : 0)) return false;
  if (epi) {
    const int row = mt * 128 + (warp & 3) * 32 + lane;
    if (op == 0) {
      s.app[row] = fmaxf(fmaxf(am[0], am[1]), fmaxf(am[2], am[3]));
    } else {
      float bbest = bb[0];
      int bidx = bi[0];
#pragma unroll
      for (int j = 1; j < 4; ++j)  // first maximum in row order: larger logit, or equal logit at a lower row
        if (bi[j] >= 0 && (bidx < 0 || bb[j] > bbest || (bb[j] == bbest && bi[j] < bidx))) {
          bbest = bb[j];
          bidx = bi[j];
        }
      if (bidx >= 0 && (s.idx[row] < 0 || bbest > s.best[row])) {
        s.best[row] = bbest;
        s.idx[row] = bidx;
      }
    }
  }
  __syncthreads();
  return true;
}

// Where the attention view (k_attn / v_attn rows) of the memory lives.
//   in place (decode, short prompts): row r of the memory is row r of `k` / `v`;  `cur` == nullptr
//   pool (prefill): every refreshed or appended row is written to a fresh pool row, `cur[r]` (shared
//   memory) names the pool row currently holding memory row r, and after the update `ver_idx`
//   receives a copy of `cur` -- a "version" of the memory costs S integers instead of S rows, and
//   block attention reads old versions through these tables while the chain runs ahead.
struct ViewStore {
  bf16* k;
  bf16* v;
  int* cur;       // shared memory [capacity] or null
  int* ver_idx;   // global [S_after] table to write after this update, or null
  int pool_next;  // first free pool row (pool mode)
};

// One full update of one kv row.  With SB the block is staged in shared memory; otherwise `pk_scr`
// ([C][D] bf16 global scratch private to this block) holds the prepared keys and values are read from
// their source.  `route_out` ([C] int32, may be null) receives the decision for every token.
// Requires C <= NT.
// PKR: `src.k` already holds prepared keys (a parallel pre-pass ran the LayerNorm), phase 1 is skipped.
template <int D, int NT, bool SB, bool PKR = false>
__device__ void memory_update(const LayerDev& L, const TokenSrc& src, const MemoryRowPtrs& mem, ViewStore& view, int capacity,
                              int S_before, int n_append, bf16* pk_scr, int* route_out, UpdateSmem<D>& s, int nc = 1,
                              int crank = 0) {
  constexpr int CPR = D / 8;
  constexpr int PST = D + 8;
  constexpr int GL = 8;                 // lanes per row in the row-parallel phases
  constexpr int GROUPS = NT / GL;
  const int C = L.C;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gl = tid % GL, grp = tid / GL;
  const int S_after = S_before + n_append;
  const int n_merge = C - n_append;
  const bool pool = view.cur != nullptr;
  // this CTA scans the tiles [crank, crank+1) * n_tiles / nc of the old memory
  const int n_tiles_all = (S_before + kScanTile - 1) / kScanTile;
  const int scan_b = min(S_before, (crank * n_tiles_all / nc) * kScanTile);
  const int scan_e = min(S_before, ((crank + 1) * n_tiles_all / nc) * kScanTile);
  // routing scan of the old memory on tcgen05: the prepared keys are staged in the swizzled operand layout, the
  // gated operand borrows the value staging area (the values are fetched after the scan)
  bool use_tc = false;
  if constexpr (SB && PKR && D == 128 && NT == 512) use_tc = s.use_tc && (C == 128 || C == 256) && n_merge > 0;
  const bool defer_v = use_tc;
  int tiles_in_flight = 0;
  // ---- 0. bring the block in: keys first (needed at once), values behind them
  BlockView blk;
  blk.g = s.g_s;
  blk.swz_rows = 0;
  if constexpr (SB) {
    if (use_tc) {
      unsigned char* dst = reinterpret_cast<unsigned char*>(s.pk_s);
      for (int c = tid; c < C * CPR; c += NT) {
        const int r = c / CPR, cc = c % CPR;
        cp_async16(dst + (size_t)(cc >> 3) * C * 128 + r * 128 + (((cc & 7) ^ (r & 7)) << 4),
                   src.k + (long long)r * src.k_st + cc * 8, 16);
      }
      cp_async_commit();
      if constexpr (D == 128 && NT == 512) {  // the first two memory tiles of the scan travel behind the keys
        const int n_t = (scan_e - scan_b + kTcTile - 1) / kTcTile;
        tiles_in_flight = min(2, max(n_t, 0));
        for (int it = 0; it < tiles_in_flight; ++it) scan_tc_load_tile<D, NT>(s, view.k, view.cur, scan_b, scan_e, it);
      }
      cp_async_commit();
      blk.swz_rows = C;
    } else {
      for (int c = tid; c < C * CPR; c += NT) {
        const int r = c / CPR, cc = c % CPR;
        cp_async16(s.pk_s + (size_t)r * PST + cc * 8, src.k + (long long)r * src.k_st + cc * 8, 16);
      }
      cp_async_commit();
      for (int c = tid; c < C * CPR; c += NT) {
        const int r = c / CPR, cc = c % CPR;
        cp_async16(s.v_s + (size_t)r * D + cc * 8, src.v + (long long)r * src.v_st + cc * 8, 16);
      }
      cp_async_commit();
    }
    blk.pk = s.pk_s; blk.pk_st = PST; blk.v = s.v_s; blk.v_st = D;
  } else {
    blk.pk = pk_scr; blk.pk_st = D; blk.v = src.v; blk.v_st = src.v_st;
  }
  for (int i = tid; i < C; i += NT) {
    s.g_s[i] = __bfloat162float(src.g[(long long)i * src.g_st]);
    s.app[i] = -INFINITY;
    s.best[i] = -INFINITY;
    s.idx[i] = -1;
    s.pos[i] = 0;
    s.flag[i] = (n_merge == 0) ? 1 : 0;
  }
  if (tid < 36) s.counters[tid] = 0;
  if (src.next_k != nullptr) {  // warm L2 with the block the next update of this row consumes
    constexpr int LPRW = D * 2 / 128 > 0 ? D * 2 / 128 : 1;  // 128-byte lines per row
    for (int c = tid; c < C * LPRW; c += NT) {
      const int r = c / LPRW, l = c % LPRW;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(src.next_k + (long long)r * src.k_st + l * 64));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(src.next_v + (long long)r * src.v_st + l * 64));
    }
  }
  if constexpr (SB) cp_async_wait<1>();
  __syncthreads();

  // ---- 1. prepared keys (in place in shared memory, or into the global scratch); 8 lanes per token
  if constexpr (PKR && !SB) {
    blk.pk = src.k;
    blk.pk_st = (int)src.k_st;
  }
#pragma unroll 2
  for (int base = 0; base < (PKR ? 0 : C); base += GROUPS) {
    const int tkn = base + grp;
    const bool act = tkn < C;
    const int t_ = act ? tkn : 0;
    RowVec<D, GL> r;
    if constexpr (SB) {
      prepare_key_row<D, GL>(L, r, s.pk_s + (size_t)t_ * PST, gl);
      if (act) store_row<D, GL>(r, s.pk_s + (size_t)t_ * PST, gl);
    } else {
      prepare_key_row<D, GL>(L, r, src.k + (long long)t_ * src.k_st, gl);
      if (act) store_row<D, GL>(r, pk_scr + (size_t)t_ * D, gl);
    }
  }
  __syncthreads();

  const int protected_rows = min(L.sink_len, S_after);

  // ---- 2. scores against the old memory, append selection
  if (n_merge > 0) {
    bool scanned = false;
    if constexpr (SB && PKR && D == 128 && NT == 512) {
      if (use_tc) {
        scanned = scan_memory_tc<D, NT>(blk, L.gate_keys != 0, C, view.k, view.cur, scan_b, scan_e, n_append > 0, protected_rows,
                                        s, tiles_in_flight);
        if (!scanned) {  // report, and stay on the warp-level path for the rest of this kernel
          if (tid == 0 && s.status) atomicExch(s.status, KVM_ERR_DEVICE_TIMEOUT);
          s.use_tc = false;
        }
      }
    }
    if (!scanned)
      scan_memory<D, NT>(blk, L.gate_keys != 0, C, view.k, view.cur, scan_b, scan_e, n_append > 0, protected_rows, s);
    if constexpr (SB) {
      if (defer_v) {  // the value staging area is free again: fetch the block's values behind the ranking
        for (int c = tid; c < C * CPR; c += NT) {
          const int r = c / CPR, cc = c % CPR;
          cp_async16(s.v_s + (size_t)r * D + cc * 8, src.v + (long long)r * src.v_st + cc * 8, 16);
        }
        cp_async_commit();
      }
    }
    if (nc > 1) {
      // all-gather of the partial results through distributed shared memory, then a local combine
      for (int i = tid; i < C * nc; i += NT) {
        const int peer = i / C, tkn = i % C;
        st_peer_f32(peer_smem_addr(s.xapp + crank * C + tkn, peer), s.app[tkn]);
        st_peer_f32(peer_smem_addr(s.xbest + crank * C + tkn, peer), s.best[tkn]);
        st_peer_s32(peer_smem_addr(s.xidx + crank * C + tkn, peer), s.idx[tkn]);
      }
      cluster_sync_all();
      for (int i = tid; i < C; i += NT) {
        float a = -INFINITY, bb = -INFINITY;
        int bi = -1;
        for (int c = 0; c < nc; ++c) {  // ranks hold increasing row ranges: strict > keeps the lowest row on ties
          a = fmaxf(a, s.xapp[c * C + i]);
          const int ci = s.xidx[c * C + i];
          const float cb = s.xbest[c * C + i];
          if (ci >= 0 && (bi < 0 || cb > bb)) { bb = cb; bi = ci; }
        }
        s.app[i] = a; s.best[i] = bb; s.idx[i] = bi;
      }
      __syncthreads();
    }
  }
  if (n_append == 1 && n_merge > 0) {
    // one append: the token with the lowest novelty score, lowest index among equals (= rank 0 of the
    // stable ranking below), found by a block-wide reduction instead of the O(C) count per token
    float bv = tid < C ? s.app[tid] : INFINITY;
    int bt = tid < C ? tid : 0x7fffffff;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int ot = __shfl_xor_sync(0xffffffffu, bt, off);
      if (ov < bv || (ov == bv && ot < bt)) { bv = ov; bt = ot; }
    }
    float* red_v = reinterpret_cast<float*>(s.counters + 4);   // [32] per-warp candidates (reused right below)
    int* red_t = s.tstart;                                      // [C] scratch at this point of the update
    if (lane == 0) { red_v[warp] = bv; red_t[warp] = bt; }
    __syncthreads();
    if (warp == 0) {
      bv = lane < NT / 32 ? red_v[lane] : INFINITY;
      bt = lane < NT / 32 ? red_t[lane] : 0x7fffffff;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int ot = __shfl_xor_sync(0xffffffffu, bt, off);
        if (ov < bv || (ov == bv && ot < bt)) { bv = ov; bt = ot; }
      }
      if (lane == 0) s.counters[2] = bt;
    }
    __syncthreads();
    if (tid < C) s.flag[tid] = tid == s.counters[2] ? 1 : 0;
    __syncthreads();
  } else if (n_append > 0 && n_merge > 0) {
    if (tid < C) {
      const float si = s.app[tid];
      int rank = 0;
#pragma unroll 4
      for (int u0 = 0; u0 < C; u0 += 4) {
        const float4 a = *reinterpret_cast<const float4*>(s.app + u0);
        rank += (a.x < si || (a.x == si && u0 + 0 < tid)) ? 1 : 0;
        rank += (a.y < si || (a.y == si && u0 + 1 < tid)) ? 1 : 0;
        rank += (a.z < si || (a.z == si && u0 + 2 < tid)) ? 1 : 0;
        rank += (a.w < si || (a.w == si && u0 + 3 < tid)) ? 1 : 0;
      }
      s.flag[tid] = rank < n_append ? 1 : 0;
    }
    __syncthreads();
  }
  if (n_append > 0) {
    // position of every appended token among the appended ones (token order): ballot prefix
    const int f = tid < C ? s.flag[tid] : 0;
    const unsigned bal = __ballot_sync(0xffffffffu, f != 0);
    if (lane == 0) s.counters[4 + warp] = __popc(bal);
    if constexpr (SB) cp_async_wait<0>();  // the values of the block have landed
    __syncthreads();
    if (tid < C) {
      int p = __popc(bal & ((1u << lane) - 1u));
      for (int w = 0; w < warp; ++w) p += s.counters[4 + w];
      s.pos[tid] = p;
      if (f) s.list[p] = tid;  // appended tokens in token order (the list is rebuilt for the merged ones later)
    }
    __syncthreads();
    // appended rows, in token order; 8 lanes per row
    for (int base = 0; base < n_append; base += GROUPS) {
      const int p_ = base + grp;
      const bool act = p_ < n_append && (S_before + p_) < capacity && (p_ % nc == crank);
      if (!__any_sync(0xffffffffu, act)) continue;  // no row for this warp (the refresh uses group shuffles: whole warps only)
      const int t_ = s.list[p_ < n_append ? p_ : 0];
      const int row = act ? S_before + p_ : 0;
      RowVec<D, GL> kr, vr;
      load_pk_row<D, GL>(kr, blk, t_, gl);
      load_row<D, GL>(vr, blk.v + (long long)t_ * blk.v_st, gl);
      if (L.gate_appends) {
        const float gt = s.g_s[t_];
#pragma unroll
        for (int i = 0; i < D / GL; ++i) {
          if (L.gate_keys) kr.x[i] = bf16_round(kr.x[i] * gt);
          if (L.gate_values) vr.x[i] = bf16_round(vr.x[i] * gt);
        }
      }
      const float vl = row_norm<D, GL>(vr);
      const int slot = pool ? view.pool_next + s.pos[t_] : row;
      if (act) {
        store_row<D, GL>(kr, mem.k_sum + (size_t)row * D, gl);
        store_row<D, GL>(vr, mem.v_sum + (size_t)row * D, gl);
        if (gl == 0) mem.vlen[row] = vl;
      }
      refresh_memory_row<D, GL>(L, kr, vr, vl, view.k + (size_t)slot * D, view.v + (size_t)slot * D, gl, act);
    }
    if (pool) {
      for (int i = tid; i < n_append; i += NT)
        if (S_before + i < capacity) view.cur[S_before + i] = view.pool_next + i;
      view.pool_next += n_append;
    }
    __syncthreads();
    if (nc > 1) cluster_sync_all();  // the appended rows written by the other CTAs are visible
  } else {
    if constexpr (SB) cp_async_wait<0>();
  }
  if (n_merge == 0) {
    if (route_out && crank == 0)
      for (int i = tid; i < C; i += NT) route_out[i] = -(1 + S_before + s.pos[i]);
    if (view.ver_idx && crank == 0)
      for (int i = tid; i < S_after; i += NT) view.ver_idx[i] = view.cur[i];
    __syncthreads();
    return;
  }

  // ---- 3. merge targets among the rows that were just appended (append-before-merge)
  if (n_append > 0 && n_append <= kDirectRows) {
    // few new rows: fp32 dot products of every token's gated key with them, 8 lanes per token (fixed
    // summation order), instead of a tensor-core pass; a new row wins only with a strictly larger logit
    for (int r = max(S_before, protected_rows); r < S_after; ++r) {
      const int slot = pool ? view.cur[r] : r;
      RowVec<D, GL> mr;  // this lane's 16 elements of the new row (one global read per row)
      load_row<D, GL>(mr, view.k + (size_t)slot * D, gl);
      for (int base = 0; base < C; base += GROUPS) {
        const int tkn = base + grp;
        const bool act = tkn < C;
        const int t_ = act ? tkn : 0;
        RowVec<D, GL> kr;
        load_pk_row<D, GL>(kr, blk, t_, gl);
        float acc = 0.f;
        if (L.gate_keys) {
          const float gt = s.g_s[t_];
#pragma unroll
          for (int i = 0; i < D / GL; ++i) acc = fmaf(bf16_round(kr.x[i] * gt), mr.x[i], acc);
        } else {
#pragma unroll
          for (int i = 0; i < D / GL; ++i) acc = fmaf(kr.x[i], mr.x[i], acc);
        }
        acc = group_sum<GL>(acc);
        if (act && gl == 0 && (s.idx[t_] < 0 || acc > s.best[t_])) {
          s.best[t_] = acc;
          s.idx[t_] = r;
        }
      }
    }
    __syncthreads();
  } else if (n_append > 0) {
    scan_memory<D, NT>(blk, L.gate_keys != 0, C, view.k, view.cur, S_before, S_after, false, protected_rows, s);
  }

  // ---- 4. group the merged tokens by target row, token order inside a group
  if (tid < C && s.flag[tid]) s.idx[tid] = -1;
  __syncthreads();
  bool is_leader = false;
  int ltok = 0;  // the token this thread leads (valid if is_leader)
  {
    // per merged token: how many tokens with the same target come before it, how many there are, which is
    // the first.  With 2C <= NT two threads share a token, each counting over one half of the block.
    const bool pair = 2 * C <= NT;
    const int tok = pair ? tid >> 1 : tid;
    const int half = pair ? tid & 1 : 0;
    const int lo = pair ? half * (C / 2) : 0, hi = pair ? lo + C / 2 : C;
    const int mine = tok < C ? s.idx[tok] : -1;
    int before = 0, total = 0, first = C;
    if (mine >= 0) {
#pragma unroll 4
      for (int u0 = lo; u0 < hi; u0 += 4) {
        const int4 a = *reinterpret_cast<const int4*>(s.idx + u0);
        const int e0 = a.x == mine, e1 = a.y == mine, e2 = a.z == mine, e3 = a.w == mine;
        total += e0 + e1 + e2 + e3;
        before += (e0 & (u0 + 0 < tok)) + (e1 & (u0 + 1 < tok)) + (e2 & (u0 + 2 < tok)) + (e3 & (u0 + 3 < tok));
        if (e3 && u0 + 3 < first) first = u0 + 3;
        if (e2 && u0 + 2 < first) first = u0 + 2;
        if (e1 && u0 + 1 < first) first = u0 + 1;
        if (e0 && u0 + 0 < first) first = u0 + 0;
      }
    }
    if (pair) {
      total += __shfl_xor_sync(0xffffffffu, total, 1);
      before += __shfl_xor_sync(0xffffffffu, before, 1);
      first = min(first, __shfl_xor_sync(0xffffffffu, first, 1));
    }
    if (mine >= 0 && half == 0) {
      s.ord[tok] = before;
      s.lead[tok] = first;
      if (before == 0) {
        s.tcnt[tok] = total;
        s.tstart[tok] = atomicAdd(&s.counters[0], total);
        is_leader = true;
        ltok = tok;
      }
    }
  }
  {  // touched rows in token order of their first token: the same order in every CTA of a cluster
    const unsigned bal = __ballot_sync(0xffffffffu, is_leader);
    if (lane == 0) s.counters[4 + warp] = __popc(bal);
    __syncthreads();
    int p = __popc(bal & ((1u << lane) - 1u)), tot = 0;
    for (int w = 0; w < NT / 32; ++w) {
      const int c = s.counters[4 + w];
      if (w < warp) p += c;
      tot += c;
    }
    if (is_leader) s.touched[p] = ltok;
    if (tid == 0) s.counters[1] = tot;
  }
  __syncthreads();
  if (tid < C) {
    if (s.idx[tid] >= 0) s.list[s.tstart[s.lead[tid]] + s.ord[tid]] = tid;
    if (route_out && crank == 0) route_out[tid] = s.flag[tid] ? -(1 + S_before + s.pos[tid]) : s.idx[tid];
  }
  __syncthreads();

  // ---- 5. fixed-order accumulation into the touched rows and refresh of their attention view;
  //         eight lanes per row; the first half of the block does the key rows, the second half the values
  const int n_touched = s.counters[1];
  {
    constexpr int HG = GROUPS / 2;
    const bool is_v = grp >= HG;
    const int hgrp = grp % HG;
    for (int base = 0; crank + nc * base < n_touched; base += HG) {  // trip count uniform: the refresh uses shuffles
      const int i = crank + nc * (base + hgrp);  // this CTA takes every nc-th touched row
      const bool act = i < n_touched;
      const int lt = s.touched[act ? i : 0];
      const int row = s.idx[lt];
      const int n = act ? s.tcnt[lt] : 0;
      const int b0 = s.tstart[lt];
      const int slot = pool ? view.pool_next + i : row;
      bf16* sum_row = (is_v ? mem.v_sum : mem.k_sum) + (size_t)row * D;
      RowVec<D, GL> sum, acc;
      load_row<D, GL>(sum, sum_row, gl);  // issued first: its latency hides behind the accumulation
      const float vl = is_v ? mem.vlen[row] : 0.f;
#pragma unroll
      for (int e = 0; e < D / GL; ++e) acc.x[e] = 0.f;
      if (!is_v) {
        for (int j = 0; j < n; ++j) {
          const int tkn = s.list[b0 + j];
          accumulate_pk_row<D, GL>(acc, blk, tkn, gl, L.gate_keys != 0, s.g_s[tkn]);
        }
      } else {
        for (int j = 0; j < n; ++j) {
          const int tkn = s.list[b0 + j];
          accumulate_row<D, GL>(acc, blk.v + (long long)tkn * blk.v_st, gl, L.gate_values != 0, s.g_s[tkn]);
        }
      }
#pragma unroll
      for (int e = 0; e < D / GL; ++e) sum.x[e] = bf16_round(sum.x[e] + bf16_round(acc.x[e]));
      if (act) store_row<D, GL>(sum, sum_row, gl);
      if (!is_v) {
        layer_norm_row<D, GL>(sum, L.ln_w, L.ln_b, L.ln_eps, gl);
        if (act) store_row<D, GL>(sum, view.k + (size_t)slot * D, gl);
      } else {
        const float nrm = fmaxf(row_norm<D, GL>(sum), 1e-12f);
        divide_by(sum.x, nrm);
#pragma unroll
        for (int e = 0; e < D / GL; ++e) sum.x[e] *= vl;
        if (act) store_row<D, GL>(sum, view.v + (size_t)slot * D, gl);
      }
    }
  }
  __syncthreads();
  if (pool) {
    for (int i = tid; i < n_touched; i += NT) view.cur[s.idx[s.touched[i]]] = view.pool_next + i;
    view.pool_next += n_touched;
    __syncthreads();
    if (view.ver_idx && crank == 0)
      for (int i = tid; i < S_after; i += NT) view.ver_idx[i] = view.cur[i];
  }
  __syncthreads();
  if (nc > 1) cluster_sync_all();  // rows refreshed by the other CTAs are visible before the next update scans them
}

}  // namespace kvm
