// Decode kernels: one new token for each of `batch` sequences with ragged lengths.
//   kvm_decode_pre_kernel   per kv row: memory update for sequences whose window start jumps at this
//                           token (one full block leaves the window), direct memory append while the
//                           sequence is shorter than one block, then the ring write of the new token
//   kvm_decode_attn_kernel  persistent joint attention over [memory ; window]: every CTA streams an equal
//                           share of all (sequence, kv head, chunk) triples with 16-byte asynchronous
//                           copies; rows cut by a share boundary are combined by their last CTA, the
//                           last CTA of the launch advances the sequences' lengths
// Follows model/kvm_mixer.py:572-713 (eager single-token step).
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "kvm_update.cuh"
#include "kvm_tc.cuh"
#include "kvm_tma_host.cuh"

namespace kvm {

__device__ __forceinline__ int bswa_begin_dev(int total, int C, int W) {
  const int end = ((total + C - 1) / C) * C;
  return max(0, end - W * C);
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start
// while its predecessor in the stream still runs; pdl_wait() returns once the predecessor has completed
// and its writes are visible (at once if the launch did not carry the attribute); pdl_trigger() lets the
// successor start early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------------------------------- pre
template <int D, int NT, bool UPDATE, bool SB>
__global__ void __launch_bounds__(NT, 1)
kvm_decode_pre_kernel(LayerDev L, DecodeCacheDev cache, Tensor4 k, Tensor4 v, Tensor4 gate,
                      const int* __restrict__ n_append_arr, bf16* pk_scr, int* route, int scope, int batch, int nc) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // `nc` CTAs (a thread-block cluster) share one kv row of a memory update: each scans its part of the memory and
  // refreshes its share of the touched rows; rank 0 alone writes the new token
  const int cta = (int)blockIdx.x / nc, crank = (int)blockIdx.x % nc;
  int row = cta;
  if (scope == 2) {
    // Only the sequences with a memory update at this token, on a grid of just their rows (a CTA of this variant
    // takes a whole SM: a grid over all rows would queue hundreds of CTAs that return at once behind the few SMs
    // the attention of the other sequences leaves free): CTA j * Hkv + h belongs to the j-th updating sequence.
    const int j = cta / L.Hkv;
    int found = -1, cnt = 0;
    for (int i = 0; i < batch && found < 0; ++i)
      if (n_append_arr[i] >= 0 && cnt++ == j) found = i;
    if (found < 0) return;
    row = found * L.Hkv + cta % L.Hkv;
  }
  const int b = row / L.Hkv, h = row % L.Hkv;
  pdl_wait();     // the previous token's attention kernel has advanced the lengths
  pdl_trigger();  // this token's attention kernel may set itself up meanwhile
  if (scope == 1) {  // only sequences without a memory update at this token
    const int na = n_append_arr ? n_append_arr[b] : -1;
    if (na >= 0) return;
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = L.C, WC = L.W * L.C;
  const int past = cache.total_len[b];
  const int S = cache.state_len[b];
  const int cap = cache.mem.capacity;

  MemoryRowPtrs m;
  m.k_sum = cache.mem.k_sum + (size_t)row * cap * D;
  m.v_sum = cache.mem.v_sum + (size_t)row * cap * D;
  m.vlen = cache.mem.vlen + (size_t)row * cap;
  m.k_attn = cache.mem.k_attn + (size_t)row * cap * D;
  m.v_attn = cache.mem.v_attn + (size_t)row * cap * D;
  bf16* rk = cache.ring_k + (size_t)row * WC * D;
  bf16* rv = cache.ring_v + (size_t)row * WC * D;
  bf16* rg = cache.ring_g + (size_t)row * WC;

  if constexpr (UPDATE) {
    const int n_app = n_append_arr ? n_append_arr[b] : -1;
    if (n_app >= 0) {
      // the block [old_begin, old_begin + C) leaves the window (model/kvm_mixer.py:646-669)
      UpdateSmem<D> s;
      s.carve(smem_raw, C, cap, SB);
      const int old_begin = bswa_begin_dev(past, C, L.W);
      const int slot0 = old_begin % WC;
      TokenSrc src;
      src.k = rk + (size_t)slot0 * D; src.k_st = D;
      src.v = rv + (size_t)slot0 * D; src.v_st = D;
      src.g = rg + slot0; src.g_st = 1;
      src.next_k = nullptr; src.next_v = nullptr;
      ViewStore view;  // decode keeps one live copy of the attention view: rows are refreshed in place
      view.k = m.k_attn; view.v = m.v_attn; view.cur = nullptr; view.ver_idx = nullptr; view.pool_next = 0;
      memory_update<D, NT, SB>(L, src, m, view, cap, S, n_app, pk_scr + (size_t)row * C * D,
                               route ? route + (size_t)row * C : nullptr, s, nc, crank);
    }
  }
  // the new token (behind the update: its ring slot may be one the leaving block has just been read from; with a
  // cluster the update ends with a cluster-wide barrier, so every CTA has read the block by now)
  if (warp == 0 && crank == 0) {
    const bf16* kp = k.row(b, h, 0);
    const bf16* vp = v.row(b, h, 0);
    const bf16 gt = *gate.row(b, h, 0);
    RowVec<D> kr, vr;
    load_row<D>(kr, kp, lane);
    load_row<D>(vr, vp, lane);
    const int slot = past % WC;
    store_row<D>(kr, rk + (size_t)slot * D, lane);
    store_row<D>(vr, rv + (size_t)slot * D, lane);
    if (lane == 0) rg[slot] = gt;
    if (past < C && S == past && past < cap) {
      // still inside the first block: the token becomes memory row `past` directly
      // (model/kvm_mixer.py:623-638; no gating on this path)
      RowVec<D> pk;
      prepare_key_row<D>(L, pk, kp, lane);
      const float vl = row_norm<D>(vr);
      store_row<D>(pk, m.k_sum + (size_t)past * D, lane);
      store_row<D>(vr, m.v_sum + (size_t)past * D, lane);
      if (lane == 0) m.vlen[past] = vl;
      refresh_memory_row<D>(L, pk, vr, vl, m.k_attn + (size_t)past * D, m.v_attn + (size_t)past * D, lane);
    }
  }
}

// ------------------------------------------------------------------------------------- attention
constexpr int kDecUpdateCluster = 2;                       // CTAs per kv row of a boundary update on the side stream
constexpr int kDecConsumers = 8;                           // math warps (16 keys of every chunk each)
constexpr int kDecThreads = (kDecConsumers + 1) * 32;      // + one producer warp
constexpr int kDecChunk = kDecConsumers * 16;              // rows per pipeline stage
constexpr int kDecBoxRows = 16;                            // rows per TMA box: the fetch granularity of a run's tail
constexpr int kDecMaxBatch = 1024;                         // sequences per launch (their chunk table lives in shared memory)
constexpr int kDecMaxSmem = 227 * 1024;   // dynamic shared memory one CTA may use (one CTA per SM)

// Shared-memory layout of the attention kernel (byte offsets), for G query heads per kv head.
// A stage holds the K rows and the V rows of one chunk as TMA boxes: for D >= 64, D/64 blocks of
// [chunk rows][64 elements] in the 128-byte swizzle (16-byte piece c of row r at position c ^ (r % 8));
// for D = 32 plain rows of 64 bytes.
struct DecSmem {
  size_t stages, stage_bytes, qst, ored, wred, meta, bars, temps, seq, total;
  __host__ __device__ DecSmem(int D, int G, int Hq, int nb, int ST) {
    size_t off = 0;
    stage_bytes = (size_t)2 * kDecChunk * D * 2;
    stages = off; off += (size_t)ST * stage_bytes;                   // 1024-byte aligned (swizzle atoms)
    qst = off;    off += (size_t)ST * G * (D + 8) * 2;               // [stage][query head][padded D] bf16
    ored = off;   off += (size_t)kDecConsumers * G * D * 4;          // [warp][query head][D] fp32
    wred = off;   off += (size_t)2 * kDecConsumers * 16 * 4;         // per-warp running max / sum
    meta = off;   off += (size_t)ST * 32;                            // per-stage chunk description (8 ints)
    bars = off;   off += (size_t)(2 * ST + 1) * 8;                   // full[ST], empty[ST], rendezvous
    temps = off;  off += (size_t)2 * Hq * 4;                         // folded softmax scales per query head
    seq = off;    off += (size_t)(3 * nb + 4) * 4;                   // per sequence: S, total, chunk prefix
    total = (off + 15) & ~(size_t)15;
  }
};

// Chunk geometry of one sequence's kv rows: up to three contiguous runs (memory rows, window part up to
// the end of the ring, wrapped window part), each cut into chunks of kDecChunk rows.
struct DecGeo {
  int S_act, slot0, len_a, len_b, c_mem, c_a, c_b;
  __device__ __forceinline__ int chunks() const { return c_mem + c_a + c_b; }
};
__device__ __forceinline__ DecGeo dec_geometry(int S, int total, int C, int W) {
  DecGeo g;
  const int WC = W * C;
  const int new_begin = bswa_begin_dev(total, C, W);
  g.S_act = new_begin > 0 ? S : 0;
  const int n_win = total - new_begin;
  g.slot0 = new_begin % WC;
  g.len_a = min(n_win, WC - g.slot0);
  g.len_b = n_win - g.len_a;
  g.c_mem = (g.S_act + kDecChunk - 1) / kDecChunk;
  g.c_a = (g.len_a + kDecChunk - 1) / kDecChunk;
  g.c_b = (g.len_b + kDecChunk - 1) / kDecChunk;
  return g;
}

// The four row arrays of the decode cache as 2-D tensors [all rows][D] with boxes of kDecBoxRows rows.
struct DecMaps {
  CUtensorMap mem_k, mem_v, ring_k, ring_v;
};

// byte offset of the 16-byte piece j of row r inside the K (or V) part of a stage
template <int D>
__device__ __forceinline__ uint32_t dec_piece(int r, int j) {
  if constexpr (D >= 64) return (uint32_t)((j >> 3) * (kDecChunk * 128) + r * 128 + (((j & 7) ^ (r & 7)) << 4));
  else return (uint32_t)(r * (D * 2) + j * 16);
}

// Bounded wait that also gives up when another warp of the CTA has given up.
__device__ __forceinline__ bool dec_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < tc::kSpinLimit; ++i) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if (i >= 8) {
      if (*abort_flag) return false;
      __nanosleep(i < 64 ? 32 : 200);
    }
  }
  return false;
}

// Joint attention of one new token per sequence over [memory ; window], persistent and bandwidth-bound.
// All (sequence, kv head, chunk) triples of the launch form one flat list (sequence-major); every CTA
// (one per SM) takes an equal contiguous range of it.  A producer warp streams the range through a ring
// of ST shared-memory stages with tiled TMA copies (boxes of 16 rows, so that the ragged end of a run
// costs at most 15 rows of extra traffic) and runs ahead of the math across row boundaries; eight math
// warps follow through full/empty mbarriers without block-wide barriers.
// Warp-level MMAs with the keys on the M dimension (each math warp owns 16 keys of every chunk) and the
// query heads of the kv head (G <= 16) on the N dimension, so that a kv head with few query heads costs
// one 8-wide tile; each warp keeps a running (max, sum, output) that is merged across the warps when the
// CTA leaves the kv row.  A row that lies inside one CTA's range is finished there; a row cut by a range
// boundary leaves partial results [m, l, acc[D]] (fp32) and the last of its CTAs combines them.  The last
// CTA of the launch advances the lengths of the sequences it covered (nobody reads them any more by then).
// Every wait is bounded; a wait that runs out sets the status word and the CTA drains.
// `mode`: 0 = all sequences, 1 = only sequences without a memory update at this token, 2 = only those with.
template <int D, int ST, int NH>
__global__ void __launch_bounds__(kDecThreads, 1)
kvm_decode_attn_kernel(LayerDev L, DecodeCacheDev cache, Tensor4 q, const int* __restrict__ n_append_arr,
                       float* __restrict__ partial, int* __restrict__ row_counters, int* __restrict__ done_counter,
                       int* __restrict__ status, bf16* __restrict__ out, float sm_scale, int b0, int nb, int nslots,
                       int per_min, int mode, const __grid_constant__ DecMaps maps) {
  constexpr int STRQ = D + 8;  // padded query rows: conflict-free fragment loads
  constexpr int KS = D / 16;   // k-steps of K Q^T
  constexpr int CH = kDecChunk, NW = kDecConsumers;
  constexpr int CPR = D / 8;                          // 16-byte pieces per row
  constexpr int BOXW = D >= 64 ? 64 : D;              // box width in elements
  constexpr int NBLK = D / BOXW;                      // boxes side by side per row group
  constexpr uint32_t kBoxBytes = (uint32_t)kDecBoxRows * BOXW * 2;
  extern __shared__ __align__(1024) unsigned char dsm_raw[];
  unsigned char* smem_raw = dsm_raw;
  const int G = L.Hq / L.Hkv, Hkv = L.Hkv;
  const DecSmem lay(D, G, L.Hq, nb, ST);
  unsigned char* stage0 = smem_raw + lay.stages;
  bf16* qst = reinterpret_cast<bf16*>(smem_raw + lay.qst);
  float* ored = reinterpret_cast<float*>(smem_raw + lay.ored);
  float* wmax = reinterpret_cast<float*>(smem_raw + lay.wred);
  float* wsum = wmax + NW * 16;
  int* meta = reinterpret_cast<int*>(smem_raw + lay.meta);            // [ST][8]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + lay.bars);  // [ST] chunk landed (transaction bytes)
  uint64_t* empty = full + ST;                                        // [ST] chunk consumed (one arrival per math warp)
  uint64_t* fbar = empty + ST;                                        // rendezvous of the math warps
  float* temp_mem = reinterpret_cast<float*>(smem_raw + lay.temps);   // [Hq]
  float* temp_win = temp_mem + L.Hq;                                  // [Hq]
  int* sq_S = reinterpret_cast<int*>(smem_raw + lay.seq);             // [nb]
  int* sq_tot = sq_S + nb;                                            // [nb]
  int* cpre = sq_tot + nb;                                            // [nb + 1] chunks per kv row, prefix
  __shared__ int s_flag, s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int C = L.C, W = L.W, WC = L.W * L.C;
  const int cap = cache.mem.capacity;

  // ---- setup: barriers, lengths of the sequences in scope, their chunk counts, the prefix over sequences
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < ST; ++s) {
      tc::mbar_init(&full[s], 1);
      tc::mbar_init(&empty[s], NW);
    }
    tc::mbar_init(fbar, NW);
    tc::fence_barrier_init();
    s_abort = 0;
    cpre[0] = 0;
  }
  for (int b = tid; b < nb; b += kDecThreads) {
    const int B = b0 + b;
    const int n_app = n_append_arr ? n_append_arr[B] : -1;
    const bool in_scope = mode == 0 || (mode == 1 && n_app < 0) || (mode == 2 && n_app >= 0);
    int cnt = 0, S = 0, total = 0;
    if (in_scope) {
      const int past = cache.total_len[B];
      S = cache.state_len[B] + (n_app > 0 ? n_app : 0);
      if (past < C && S == past) S += 1;  // direct append done by the pre kernel
      total = past + 1;
      cnt = dec_geometry(S, total, C, W).chunks();
    }
    sq_S[b] = S;
    sq_tot[b] = total;
    cpre[b + 1] = cnt;
  }
  for (int h = tid; h < L.Hq; h += kDecThreads) {
    temp_mem[h] = sm_scale * L.state_temp[h] * kLog2e;
    temp_win[h] = sm_scale * L.front_temp[h] * kLog2e;
  }
  __syncthreads();
  if (warp == 0) {  // inclusive scan of cpre[1..nb], 32 entries at a time
    int carry = 0;
    for (int base = 0; base < nb; base += 32) {
      const int i = base + lane;
      int x = i < nb ? cpre[i + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
      }
      if (i < nb) cpre[i + 1] = x + carry;
      carry += __shfl_sync(0xffffffffu, x, 31);
    }
  }
  __syncthreads();
  const int total_f = cpre[nb] * Hkv;                         // chunks of the launch
  const int per = max(per_min, (total_f + (int)gridDim.x - 1) / (int)gridDim.x);
  const int active = (total_f + per - 1) / per;               // CTAs with work
  const int cta = blockIdx.x;
  // CTAs without a share of the list still take part in the launch counter below: the lengths may only move
  // once every CTA of the grid has read them
  const bool has_work = cta < active;
  const int f_begin = has_work ? cta * per : 0, f_end = has_work ? min(total_f, f_begin + per) : 0;
  const int nloc = f_end - f_begin;
  volatile int* abort_flag = &s_abort;
  pdl_trigger();  // the next token's ring-write kernel may be staged (it waits for this grid to complete)

  if (!has_work) {
    // nothing to stream
  } else if (warp == NW) {
    // =============================================================== producer warp (lanes in lockstep)
    int pb, ph, pc, pcb;
    DecGeo pg;
    {
      int lo = 0, hi = nb - 1;  // last b with cpre[b] * Hkv <= f_begin: its chunk range holds f_begin
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (cpre[mid] * Hkv <= f_begin) lo = mid; else hi = mid - 1;
      }
      pb = lo;
      pcb = cpre[pb + 1] - cpre[pb];
      const int rem = f_begin - cpre[pb] * Hkv;
      ph = rem / pcb;
      pc = rem - ph * pcb;
      pg = dec_geometry(sq_S[pb], sq_tot[pb], C, W);
    }
    pdl_wait();  // the ring rows of this token are written (everything above only needs the lengths)
    for (int i = 0; i < nloc; ++i) {
      const int s = i % ST;
      if (i >= ST) {  // the math warps are done with the chunk that used this stage
        const bool ok = dec_wait(&empty[s], (uint32_t)((i / ST - 1) & 1), abort_flag);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) {
            s_abort = 1;
            atomicExch(status, KVM_ERR_DEVICE_TIMEOUT);
          }
          break;
        }
      }
      const int row = (b0 + pb) * Hkv + ph;
      int n, y0;
      const bool is_mem = pc < pg.c_mem;
      if (is_mem) {
        n = min(CH, pg.S_act - pc * CH);
        y0 = row * cap + pc * CH;
      } else if (pc < pg.c_mem + pg.c_a) {
        const int c = pc - pg.c_mem;
        n = min(CH, pg.len_a - c * CH);
        y0 = row * WC + pg.slot0 + c * CH;
      } else {
        const int c = pc - pg.c_mem - pg.c_a;
        n = min(CH, pg.len_b - c * CH);
        y0 = row * WC + c * CH;
      }
      const bool first = i == 0 || pc == 0;
      const bool last = i == nloc - 1 || pc == pcb - 1;
      const int groups = (n + kDecBoxRows - 1) / kDecBoxRows;
      if (lane == 0) {
        int seg = 0, nsegs = 1;
        if (last) {
          const int row_f = cpre[pb] * Hkv + ph * pcb;  // flat index of the row's first chunk
          const int first_cta = row_f / per;
          seg = cta - first_cta;
          nsegs = (row_f + pcb - 1) / per - first_cta + 1;
        }
        int* m = meta + s * 8;
        m[0] = n | (is_mem ? 1 << 16 : 0) | (first ? 1 << 17 : 0) | (last ? 1 << 18 : 0) | (ph << 20);
        m[1] = row;
        m[2] = seg;
        m[3] = nsegs;
        tc::mbar_arrive_expect_tx(&full[s], (uint32_t)groups * 2u * NBLK * kBoxBytes + (first ? (uint32_t)(G * D * 2) : 0u));
      }
      __syncwarp();
      if (lane < groups) {  // one row group (16 rows of K and of V) per lane
        const CUtensorMap* mk = is_mem ? &maps.mem_k : &maps.ring_k;
        const CUtensorMap* mv = is_mem ? &maps.mem_v : &maps.ring_v;
        unsigned char* dk = stage0 + (size_t)s * lay.stage_bytes + (size_t)lane * kDecBoxRows * (BOXW * 2);
        unsigned char* dv = dk + (size_t)CH * D * 2;
        const int y = y0 + lane * kDecBoxRows;
#pragma unroll
        for (int blk = 0; blk < NBLK; ++blk) {
          tc::tma_load_2d(dk + (size_t)blk * CH * 128, mk, blk * 64, y, &full[s]);
          tc::tma_load_2d(dv + (size_t)blk * CH * 128, mv, blk * 64, y, &full[s]);
        }
      }
      if (first && lane < G)  // the query rows of this kv head travel with the first chunk of the row segment
        tc::bulk_g2s(qst + ((size_t)s * G + lane) * STRQ, q.row(b0 + pb, ph * G + lane, 0), D * 2, &full[s]);
      // advance the cursor
      if (++pc == pcb) {
        pc = 0;
        if (++ph == Hkv) {
          ph = 0;
          ++pb;
          while (pb < nb && cpre[pb + 1] == cpre[pb]) ++pb;
          if (pb < nb) {
            pcb = cpre[pb + 1] - cpre[pb];
            pg = dec_geometry(sq_S[pb], sq_tot[pb], C, W);
          }
        }
      }
    }
  } else {
    // ==================================================================================== math warps
    // Math layout: the keys are the M dimension of the MMAs (16 keys of this warp per chunk), the query heads
    // of the kv head the N dimension (NH tiles of 8 heads).  S^T = K Q^T: thread (g, t) holds keys g and g+8
    // for heads 2t, 2t+1 of each head tile; O^T = V^T P^T accumulates [d][head] with d on the M dimension.
    constexpr int DT16 = D / 16;
    uint32_t qb[NH][KS][2];            // B fragments of Q^T: head g (+8 per tile), d = 16 ks + 2t (+8)
    float scl_mem[NH][2], scl_win[NH][2];
    float m_run[NH][2], l_run[NH][2];  // running max / partial sum of heads 2t, 2t+1 (this thread's keys)
    float o[NH][DT16][4];              // [d = 16 dt + g (+8)][head 2t, 2t+1]
    const int krow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;  // ldmatrix row of the K tile
    const int vrow = warp * 16 + (lane & 7) + (lane >> 4) * 8;         // ldmatrix row of the V tile
    uint32_t fphase = 0;               // phase of the rendezvous barrier
    bool alive = true;
    // all math warps meet (bounded): false if somebody gave up
    auto rendezvous = [&]() -> bool {
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(fbar);
      const bool ok = dec_wait(fbar, fphase & 1, abort_flag);
      ++fphase;
      return __all_sync(0xffffffffu, ok);
    };

    for (int i = 0; i < nloc && alive; ++i) {
      const int s = i % ST;
      if (!__all_sync(0xffffffffu, dec_wait(&full[s], (uint32_t)((i / ST) & 1), abort_flag))) {
        alive = false;
        break;
      }
      const int4 md = *reinterpret_cast<const int4*>(meta + s * 8);
      const int n = md.x & 0xffff;
      const bool is_mem = (md.x >> 16) & 1, first = (md.x >> 17) & 1, last = (md.x >> 18) & 1;
      const int row = md.y;
      const int hkv = md.x >> 20;
      if (first) {  // new kv row (or the CTA's first chunk): reset the running state, fetch the query fragments
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          const int qh = h * 8 + g;  // head supplied by this thread to the B operand
          const bool okq = qh < G;
          const bf16* qp = qst + ((size_t)s * G + (okq ? qh : 0)) * STRQ + t * 2;
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            qb[h][ks][0] = okq ? *reinterpret_cast<const uint32_t*>(qp + ks * 16) : 0u;
            qb[h][ks][1] = okq ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8) : 0u;
          }
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int hh = h * 8 + t * 2 + j;  // head of this thread's accumulator columns
            const int hq = hkv * G + (hh < G ? hh : 0);
            scl_mem[h][j] = temp_mem[hq];
            scl_win[h][j] = temp_win[hq];
            m_run[h][j] = -INFINITY;
            l_run[h][j] = 0.f;
          }
#pragma unroll
          for (int dt = 0; dt < DT16; ++dt) o[h][dt][0] = o[h][dt][1] = o[h][dt][2] = o[h][dt][3] = 0.f;
        }
      }
      if (warp * 16 < n) {
        unsigned char* sK = stage0 + (size_t)s * lay.stage_bytes;
        unsigned char* sV = sK + (size_t)CH * D * 2;
        if (n < warp * 16 + 16) {
          // ragged end of the run inside this warp's rows: what the box brought in beyond the run is not
          // part of it; scores are masked below, values are zeroed here (0 * garbage must stay finite)
          const int r_lo = n, cnt = (warp * 16 + 16 - n) * CPR;
          for (int p = lane; p < cnt; p += 32) {
            const int r = r_lo + p / CPR, j = p % CPR;
            *reinterpret_cast<uint4*>(sV + dec_piece<D>(r, j)) = make_uint4(0, 0, 0, 0);
          }
          tc::fence_proxy_async();  // ... before a later TMA copy overwrites these bytes
          __syncwarp();
        }
        // S^T = K Q^T for this warp's 16 keys of the chunk
        float sacc[NH][4];
#pragma unroll
        for (int h = 0; h < NH; ++h) sacc[h][0] = sacc[h][1] = sacc[h][2] = sacc[h][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          uint32_t ka[4];
          ldmatrix_x4(ka, sK + dec_piece<D>(krow, ks * 2 + (lane >> 4)));
#pragma unroll
          for (int h = 0; h < NH; ++h) mma_bf16_16816(sacc[h], ka, qb[h][ks][0], qb[h][ks][1]);
        }
        const bool ok_lo = warp * 16 + g < n, ok_hi = warp * 16 + g + 8 < n;
        uint32_t pb[NH][2];
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          float mx[2], f[2];
          bool grew = false;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float sc = is_mem ? scl_mem[h][j] : scl_win[h][j];
            sacc[h][j] = ok_lo ? sacc[h][j] * sc : -INFINITY;
            sacc[h][2 + j] = ok_hi ? sacc[h][2 + j] * sc : -INFINITY;
            float x = fmaxf(sacc[h][j], sacc[h][2 + j]);
            x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 4));
            x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 8));
            x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 16));
            mx[j] = x;
            grew = grew || x > m_run[h][j];
          }
          if (__any_sync(0xffffffffu, grew)) {  // a running maximum moved: rescale what has been accumulated
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const float mn = fmaxf(m_run[h][j], mx[j]);
              f[j] = m_run[h][j] == -INFINITY ? 0.f : exp2f(m_run[h][j] - mn);
              m_run[h][j] = mn;
              l_run[h][j] *= f[j];
            }
#pragma unroll
            for (int dt = 0; dt < DT16; ++dt) {
              o[h][dt][0] *= f[0];
              o[h][dt][1] *= f[1];
              o[h][dt][2] *= f[0];
              o[h][dt][3] *= f[1];
            }
          }
          const float mu0 = m_run[h][0] == -INFINITY ? 0.f : m_run[h][0];
          const float mu1 = m_run[h][1] == -INFINITY ? 0.f : m_run[h][1];
          const float p0 = exp2f(sacc[h][0] - mu0), p1 = exp2f(sacc[h][1] - mu1);
          const float p2 = exp2f(sacc[h][2] - mu0), p3 = exp2f(sacc[h][3] - mu1);
          l_run[h][0] += p0 + p2;
          l_run[h][1] += p1 + p3;
          // [key g][heads 2t, 2t+1] -> [head g][keys 2t, 2t+1]: the B operand of O^T += V^T P^T
          pb[h][0] = movmatrix_trans(pack_bf16(p0, p1));
          pb[h][1] = movmatrix_trans(pack_bf16(p2, p3));
        }
#pragma unroll
        for (int dt = 0; dt < DT16; ++dt) {
          uint32_t va[4];
          ldmatrix_x4_trans(va, sV + dec_piece<D>(vrow, dt * 2 + ((lane >> 3) & 1)));
#pragma unroll
          for (int h = 0; h < NH; ++h) mma_bf16_16816(o[h][dt], va, pb[h][0], pb[h][1]);
        }
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&empty[s]);  // this warp is done with the stage
      if (!last) continue;

      // ---- the CTA leaves this kv row: merge the warps' running states
      const int seg = md.z, nsegs = md.w;
      const int b = row / Hkv;  // absolute sequence index
#pragma unroll
      for (int h = 0; h < NH; ++h) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float l = l_run[h][j];
          l += __shfl_xor_sync(0xffffffffu, l, 4);
          l += __shfl_xor_sync(0xffffffffu, l, 8);
          l += __shfl_xor_sync(0xffffffffu, l, 16);
          const int hh = h * 8 + t * 2 + j;
          if (hh < G) {
            if (g == 0) {
              wmax[warp * 16 + hh] = m_run[h][j];
              wsum[warp * 16 + hh] = l;
            }
            float* dst = ored + ((size_t)warp * G + hh) * D + g;
#pragma unroll
            for (int dt = 0; dt < DT16; ++dt) {
              dst[dt * 16] = o[h][dt][j];
              dst[dt * 16 + 8] = o[h][dt][2 + j];
            }
          }
        }
      }
      if (!rendezvous()) {
        alive = false;
        break;
      }
      for (int gq = 0; gq < G; ++gq) {
        const int hq = hkv * G + gq;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, wmax[w * 16 + gq]);
        float f[NW], lsum = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          f[w] = wmax[w * 16 + gq] == -INFINITY ? 0.f : exp2f(wmax[w * 16 + gq] - M);
          lsum += f[w] * wsum[w * 16 + gq];
        }
        float acc = 0.f;
        if (tid < D) {
          const float* src = ored + (size_t)gq * D + tid;
#pragma unroll
          for (int w = 0; w < NW; ++w) acc += f[w] * src[(size_t)w * G * D];
        }
        if (nsegs == 1) {  // the whole row was here
          if (tid < D) out[(size_t)b * L.Hq * D + (size_t)hq * D + tid] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
        } else {
          float* pout = partial + ((size_t)(b * L.Hq + hq) * nslots + seg) * (D + 2);
          if (tid < D) pout[2 + tid] = acc;
          if (tid == 0) {
            pout[0] = M;
            pout[1] = lsum;
          }
        }
      }
      if (nsegs > 1) __threadfence();
      if (!rendezvous()) {  // everybody has read the merge buffers (and fenced its partial results)
        alive = false;
        break;
      }
      if (nsegs > 1) {  // the last CTA of this kv row combines the partial results
        if (tid == 0) {
          const int prev = atomicAdd(&row_counters[row], 1);
          s_flag = (prev == nsegs - 1);
        }
        if (!rendezvous()) {
          alive = false;
          break;
        }
        if (s_flag) {
          __threadfence();
          for (int gq = 0; gq < G; ++gq) {
            const int hq = hkv * G + gq;
            const float* pin = partial + ((size_t)(b * L.Hq + hq) * nslots) * (D + 2);
            float M = -INFINITY;
            for (int s2 = 0; s2 < nsegs; ++s2) M = fmaxf(M, __ldcg(pin + (size_t)s2 * (D + 2)));
            if (tid < D) {
              float Lsum = 0.f, a = 0.f;
              for (int s2 = 0; s2 < nsegs; ++s2) {
                const float ms = __ldcg(pin + (size_t)s2 * (D + 2));
                const float w = ms == -INFINITY ? 0.f : exp2f(ms - M);
                Lsum += w * __ldcg(pin + (size_t)s2 * (D + 2) + 1);
                a += w * __ldcg(pin + (size_t)s2 * (D + 2) + 2 + tid);
              }
              out[(size_t)b * L.Hq * D + (size_t)hq * D + tid] = __float2bfloat16_rn(Lsum > 0.f ? a / Lsum : 0.f);
            }
          }
          if (tid == 0) row_counters[row] = 0;
        }
      }
    }
    if (!alive && lane == 0) {
      s_abort = 1;
      atomicExch(status, KVM_ERR_DEVICE_TIMEOUT);
    }
  }
  if (*abort_flag) {
    // somebody gave up: copies of this CTA may still be in flight, give them a bounded time to land
    for (int k2 = 0; k2 < 1000; ++k2) __nanosleep(1000);
  }

  // ---- the last CTA of the launch advances the lengths of the sequences in scope: by then every CTA of the
  //      grid (also those without work) has derived its geometry from the old lengths
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int prev = atomicAdd(done_counter, 1);
    s_flag = (prev == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (s_flag) {
    for (int b = tid; b < nb; b += kDecThreads) {
      if (cpre[b + 1] != cpre[b]) {
        cache.total_len[b0 + b] = sq_tot[b];
        cache.state_len[b0 + b] = sq_S[b];
      }
    }
    if (tid == 0) *done_counter = 0;
  }
}

// Rebuild the attention view of rows [0, state_len[b]) from the carried sums.
template <int D>
__global__ void kvm_memory_refresh_kernel(LayerDev L, MemoryDev mem, const int* __restrict__ state_len) {
  const int row = blockIdx.y;
  const int b = row / L.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + warp;
  if (r >= state_len[b] || r >= mem.capacity) return;
  const size_t off = ((size_t)row * mem.capacity + r) * D;
  RowVec<D> ks, vs;
  load_row<D>(ks, mem.k_sum + off, lane);
  load_row<D>(vs, mem.v_sum + off, lane);
  refresh_memory_row<D>(L, ks, vs, mem.vlen[(size_t)row * mem.capacity + r], mem.k_attn + off, mem.v_attn + off, lane);
}

// ------------------------------------------------------------------------------------- host side
constexpr int kMaxDevices = 64;  // device ordinals the per-device caches below cover

static int device_sm_count() {
  int dev = 0, n_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      n_sm <= 0)
    return 148;
  return n_sm;
}

// [rows][D] bf16 row array -> tensor map with boxes of kDecBoxRows rows x min(D, 64) elements
static bool encode_rows_map(CUtensorMap* m, const void* base, uint64_t rows, int D) {
  const cuuint64_t gdim[2] = {(cuuint64_t)D, rows};
  const cuuint64_t gstr[1] = {(cuuint64_t)D * 2};
  const cuuint32_t box[2] = {(cuuint32_t)(D >= 64 ? 64 : D), (cuuint32_t)kDecBoxRows};
  return encode_bf16_map(m, base, 2, gdim, gstr, box);
}

// The tensor maps of a decode cache (small cache keyed by the array addresses and sizes: a serving loop
// calls with the same cache every token).
static bool decode_maps(const DecodeCacheDev& c, uint64_t kv_rows, int cap, int WC, int D, DecMaps* out) {
  struct Entry {
    const void *mk, *mv, *rk, *rv;
    uint64_t kv_rows;
    int cap, WC, D;
    DecMaps maps;
  };
  static Entry cache[8];
  static int n_used = 0, next = 0;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_used; ++i) {
    const Entry& e = cache[i];
    if (e.mk == c.mem.k_attn && e.mv == c.mem.v_attn && e.rk == c.ring_k && e.rv == c.ring_v && e.kv_rows == kv_rows &&
        e.cap == cap && e.WC == WC && e.D == D) {
      *out = e.maps;
      return true;
    }
  }
  Entry e;
  e.mk = c.mem.k_attn; e.mv = c.mem.v_attn; e.rk = c.ring_k; e.rv = c.ring_v;
  e.kv_rows = kv_rows; e.cap = cap; e.WC = WC; e.D = D;
  if (!encode_rows_map(&e.maps.mem_k, c.mem.k_attn, kv_rows * (uint64_t)cap, D) ||
      !encode_rows_map(&e.maps.mem_v, c.mem.v_attn, kv_rows * (uint64_t)cap, D) ||
      !encode_rows_map(&e.maps.ring_k, c.ring_k, kv_rows * (uint64_t)WC, D) ||
      !encode_rows_map(&e.maps.ring_v, c.ring_v, kv_rows * (uint64_t)WC, D))
    return false;
  cache[next] = e;
  next = (next + 1) % 8;
  if (n_used < 8) ++n_used;
  *out = e.maps;
  return true;
}

// Side stream and events for overlapping a boundary update with the attention of the other sequences
// (created once per device, on first use).
struct DecodeSide {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool ok = false;
};
static DecodeSide* decode_side() {
  static DecodeSide side[kMaxDevices];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  DecodeSide& d = side[dev];
  if (!d.ok) {
    if (cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&d.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&d.join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    d.ok = true;
  }
  return &d;
}

// Launch with the programmatic-serialization attribute when `pdl` is set (see pdl_wait above).
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

template <int D, int ST, int NH>
static cudaError_t launch_decode_attn(const LayerDev& L, int batch, const DecodeCacheDev& cache, Tensor4 q,
                                      const int* n_append, int max_rows, bf16* out, float* partial, int* counters,
                                      int nslots, int mode, int grid, const DecMaps& maps, bool pdl, int done_slot,
                                      cudaStream_t stream) {
  // The workspace holds `nslots` partial results per query head; a kv row of at most max_chunks chunks cut
  // into ranges of at least per_min chunks never needs more.
  const int G = L.Hq / L.Hkv, rows = batch * L.Hkv;
  const int max_chunks = (max_rows + kDecChunk - 1) / kDecChunk + 3;
  const int per_min = (max_chunks + nslots - 2) / (nslots - 1);
  auto kern = kvm_decode_attn_kernel<D, ST, NH>;
  static size_t smem_set[kMaxDevices] = {0};  // largest dynamic shared memory enabled so far, per device
  static std::mutex mu;
  int dev_now = 0;
  if (cudaGetDevice(&dev_now) != cudaSuccess || dev_now < 0 || dev_now >= kMaxDevices) return cudaErrorInvalidDevice;
  for (int b0 = 0; b0 < batch; b0 += kDecMaxBatch) {
    const int nb = std::min(kDecMaxBatch, batch - b0);
    const DecSmem lay(D, G, L.Hq, nb, ST);
    {
      std::lock_guard<std::mutex> lock(mu);  // function attributes are per device
      if (lay.total > smem_set[dev_now]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lay.total);
        if (e != cudaSuccess) return e;
        smem_set[dev_now] = lay.total;
      }
    }
    cudaError_t e = launch_pdl(kern, dim3(grid), dim3(kDecThreads), lay.total, stream, pdl && batch <= kDecMaxBatch, L, cache, q,
                               n_append, partial, counters, counters + rows + done_slot, counters + rows + batch, out,
                               1.0f / sqrtf((float)D), b0, nb, nslots, per_min, mode, maps);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// `any_update`: number of sequences with a memory update at this token (0: none; any positive value is
// treated as "some" when the count is not known).  `overlap`: a boundary update may run on the library's
// side stream next to the attention of the sequences without one.
template <int D>
static cudaError_t launch_decode(const LayerDev& L, int batch, const DecodeCacheDev& cache, Tensor4 q, Tensor4 k,
                                 Tensor4 v, Tensor4 gate, const int* n_append, int any_update, int max_rows, bf16* out,
                                 int* route, bf16* pk_scr, float* partial, int* counters, int nslots,
                                 int overlap, cudaStream_t stream) {
  constexpr int NT = 512;
  const int rows = batch * L.Hkv, G = L.Hq / L.Hkv;
  if (G > 16) return cudaErrorInvalidValue;  // the query heads of a kv head form one M=16 MMA tile
  const int n_sm = device_sm_count();
  // three stages when they fit beside the reduction buffers, else two
  const bool st3 = DecSmem(D, G, L.Hq, std::min(batch, kDecMaxBatch), 3).total <= (size_t)kDecMaxSmem;
  DecMaps maps;
  if (!decode_maps(cache, (uint64_t)rows, cache.mem.capacity, L.W * L.C, D, &maps)) return cudaErrorInvalidValue;
  // `done_slot`: which launch counter of the workspace the launch uses (two launches that may run at the same
  // time need one each); `st`: the stream it goes to
  auto attn = [&](int mode, int grid, const int* na, bool pdl = false, int done_slot = 0, cudaStream_t st = nullptr) {
    if (st == nullptr) st = stream;
    if (G <= 8)
      return st3 ? launch_decode_attn<D, 3, 1>(L, batch, cache, q, na, max_rows, out, partial, counters, nslots, mode, grid, maps, pdl, done_slot, st)
                 : launch_decode_attn<D, 2, 1>(L, batch, cache, q, na, max_rows, out, partial, counters, nslots, mode, grid, maps, pdl, done_slot, st);
    return st3 ? launch_decode_attn<D, 3, 2>(L, batch, cache, q, na, max_rows, out, partial, counters, nslots, mode, grid, maps, pdl, done_slot, st)
               : launch_decode_attn<D, 2, 2>(L, batch, cache, q, na, max_rows, out, partial, counters, nslots, mode, grid, maps, pdl, done_slot, st);
  };
  cudaError_t e;
  {
    // The ring-write kernel runs between attention kernels that use nearly all shared memory of an SM:
    // give it the same shared-memory carve-out so that the SMs are not reconfigured twice per token.
    static bool carve_set[kMaxDevices] = {false};
    static std::mutex mu;
    int dev_now = 0;
    if (cudaGetDevice(&dev_now) == cudaSuccess && dev_now >= 0 && dev_now < kMaxDevices) {
      std::lock_guard<std::mutex> lock(mu);
      if (!carve_set[dev_now]) {
        cudaFuncSetAttribute(kvm_decode_pre_kernel<D, 32, false, false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             (int)cudaSharedmemCarveoutMaxShared);
        carve_set[dev_now] = true;
      }
    }
  }
  if (!any_update) {
    // plain token: the two kernels are chained with programmatic dependent launches (`overlap` callers only)
    const bool pdl = overlap != 0;
    e = launch_pdl(kvm_decode_pre_kernel<D, 32, false, false>, dim3(rows), dim3(32), 0, stream, pdl, L, cache, k, v, gate,
                   (const int*)nullptr, pk_scr, route, 0, batch, 1);
    if (e != cudaSuccess) return e;
    return attn(0, n_sm, nullptr, pdl);
  }
  const bool sb = update_block_fits_smem<D>(L.C, cache.mem.capacity);
  const size_t smem_u = UpdateSmem<D>::bytes(L.C, cache.mem.capacity, sb);
  auto upd = sb ? kvm_decode_pre_kernel<D, NT, true, true> : kvm_decode_pre_kernel<D, NT, true, false>;
  e = cudaFuncSetAttribute(upd, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_u);
  if (e != cudaSuccess) return e;
  // A cluster of CTAs per updating kv row while the updating rows are few (the update is a chain of short phases:
  // more CTAs per row shorten it, and the updated sequences' attention behind it gets their SMs)
  int nc = 1;
  for (int c = kDecUpdateCluster; c > 1; c >>= 1)
    if (any_update * L.Hkv * c * 4 <= n_sm) { nc = c; break; }
  const int upd_sms = any_update * L.Hkv * nc;  // SMs the updating rows occupy (one CTA each)
  DecodeSide* side = (overlap && any_update < batch && upd_sms * 2 <= n_sm) ? decode_side() : nullptr;
  if (!side) {  // one stream: update + ring write for every row, then attention over everything
    upd<<<rows, NT, smem_u, stream>>>(L, cache, k, v, gate, n_append, pk_scr, route, 0, batch, 1);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return attn(0, n_sm, n_append);
  }
  // fork: the updating sequences' rows on the side stream ...
  if ((e = cudaEventRecord(side->fork, stream)) != cudaSuccess) return e;
  if ((e = cudaStreamWaitEvent(side->stream, side->fork, 0)) != cudaSuccess) return e;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(upd_sms);
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = smem_u;
    cfg.stream = side->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nc;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if ((e = cudaLaunchKernelEx(&cfg, upd, L, cache, k, v, gate, n_append, pk_scr, route, 2, batch, nc)) != cudaSuccess) return e;
  }
  // ... followed there by their attention, on the SMs the update leaves (second launch counter of the workspace;
  // the two attention launches touch disjoint sequences, rows, partial slots and outputs)
  if ((e = attn(2, upd_sms, n_append, false, 1, side->stream)) != cudaSuccess) return e;
  if ((e = cudaEventRecord(side->join, side->stream)) != cudaSuccess) return e;
  // ... next to the ring write and the attention of all others, which leave those SMs free
  kvm_decode_pre_kernel<D, 32, false, false><<<rows, 32, 0, stream>>>(L, cache, k, v, gate, n_append, pk_scr, route, 1, batch, 1);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  if ((e = attn(1, n_sm - upd_sms, n_append)) != cudaSuccess) return e;
  // join
  return cudaStreamWaitEvent(stream, side->join, 0);
}

cudaError_t decode_dispatch(int D, const LayerDev& L, int batch, const DecodeCacheDev& cache, Tensor4 q, Tensor4 k,
                            Tensor4 v, Tensor4 gate, const int* n_append, int any_update, int max_rows, bf16* out,
                            int* route, bf16* pk_scr, float* partial, int* counters, int nslots, int overlap,
                            cudaStream_t stream) {
  switch (D) {
    case 32: return launch_decode<32>(L, batch, cache, q, k, v, gate, n_append, any_update, max_rows, out, route, pk_scr, partial, counters, nslots, overlap, stream);
    case 64: return launch_decode<64>(L, batch, cache, q, k, v, gate, n_append, any_update, max_rows, out, route, pk_scr, partial, counters, nslots, overlap, stream);
    case 128: return launch_decode<128>(L, batch, cache, q, k, v, gate, n_append, any_update, max_rows, out, route, pk_scr, partial, counters, nslots, overlap, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t refresh_dispatch(int D, const LayerDev& L, int batch, MemoryDev mem, const int* state_len, cudaStream_t stream) {
  dim3 grid((mem.capacity + 7) / 8, batch * L.Hkv);
  switch (D) {
    case 32: kvm_memory_refresh_kernel<32><<<grid, 256, 0, stream>>>(L, mem, state_len); break;
    case 64: kvm_memory_refresh_kernel<64><<<grid, 256, 0, stream>>>(L, mem, state_len); break;
    case 128: kvm_memory_refresh_kernel<128><<<grid, 256, 0, stream>>>(L, mem, state_len); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace kvm
