// The memory chain of the prefill for head_dim 128 and blocks of 128 or 256 tokens, organised for the latency of
// one update (the updates of a kv row are strictly sequential: block m routes against the memory block m-1 left).
//
// Follows the reference's eager update (model/kvm_mixer.py:250-340) with the fp32 merge routing of
// model/kvm_fp32_routing_reference.py:24-49; what the reference does with 3-5 host-issued launches per block
// (model/kernels/kvm_triton_training_kernels.py:1606-1747) is one resident step here.
//
// Split of the work
//   kvm_chain_tc_kernel   routing and the KEY side of the memory: a cluster of 1..8 CTAs per kv row walks all
//                         updates.  Memory row r belongs to CTA r % nc, which keeps the attention view of its
//                         rows (k_attn) RESIDENT in shared memory in the tensor-core operand layout, so a routing
//                         pass loads nothing.  Per update, in the common case of few appended rows:
//                           1. logits pass    S = gk x k_attn^T against the memory as it is (tcgen05, accumulators
//                                             in tensor memory), running fp32 first-argmax per token (sink rows
//                                             excluded), then the novelty pass S = pk x k_attn^T, running maximum
//                                             per token; both partial results exchanged between the CTAs in one
//                                             go (st.async into the peers' shared memory); the n_append tokens of
//                                             lowest bf16-rounded novelty are appended (LayerNorm by one warp per
//                                             row) and scored against every token (dot products, or a small third
//                                             MMA pass); a new row wins a token only with a strictly larger logit
//                                             (with many appended rows: novelty pass, appends, then one logits pass
//                                             against the memory after the appends)
//                           2. scatter        delta[rows x D] = onehot[rows x tokens] x gk[tokens x D] on the
//                                             tensor cores (touched rows compacted onto the 128 accumulator
//                                             lanes; the one-hot operand lives in the buffer of the prepared keys,
//                                             cleared by the copy engine; products are exact, the accumulation order
//                                             is the hardware's and fixed), then row = bf16(row + bf16(delta)),
//                                             LayerNorm refresh of the touched rows into shared memory and into the
//                                             row pool
//                         Prepared keys pk and gated keys gk = bf16(pk * gate) of every token come from a parallel
//                         pre-pass and arrive by tiled TMA, issued as soon as the scatter has read the buffers.
//                         CTAs of the launch beyond the routing's (whole clusters on the SMs it leaves free) work on
//                         the value side meanwhile: see kvm_vdelta.cuh.
//   value side            which no later update reads: value deltas per (kv row, update) on the tensor cores
//                         (kvm_vdelta.cuh), then one warp per memory row (kvm_vpass.cu); kvm_vpass_kernel below is
//                         the variant for a chain of which only the final memory is wanted (no versions): one warp
//                         per memory row walks the routing decisions of all updates and accumulates the gated
//                         values routed to its row in token order.
// Every wait is bounded; a wait that runs out sets the status word, all roles and all CTAs of the cluster leave
// through the common exit, tensor memory is freed.
#include <algorithm>
#include <mutex>

#include "kvm_common.cuh"
#include "kvm_tc.cuh"
#include "kvm_tma_host.cuh"
#include "kvm_vdelta.cuh"

namespace kvm {
namespace chain {

constexpr int HD = 128;
constexpr int kWorkerWarps = 16;
constexpr int kWorkers = kWorkerWarps * 32;   // threads that do everything but issuing copies and MMAs
constexpr int kIssuers = 2;                   // issuing threads (one warp each): issuing an MMA costs its thread about as much
                                              // as the tensor core needs to execute it, so each token tile has its own
constexpr int kThreads = kWorkers + kIssuers * 32;
constexpr int kChunk = 256;                   // memory rows per MMA instruction and per tensor-memory chunk (the N limit)
constexpr int kRowPad = 64;                   // granularity of the resident rows per CTA
constexpr int kLoaderThread = 15 * 32;        // the worker thread that issues the next block's copies
constexpr int kNewRows = 16;                  // up to this many appended rows per update take the logits-first order
constexpr int kDirectNew = 2;                 // ... and up to this many are scored with plain dot products instead of an MMA pass
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxSmem = 226 * 1024;          // dynamic part; the kernel also holds 1 KB of static shared memory

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Shared-memory carve-up (byte offsets from a 1024-byte aligned base).
struct Layout {
  int Rcap;  // resident memory rows per CTA (multiple of 64)
  uint32_t R, P, G, xbuf, part, tok, rowi, tloc, stat, bars, total;
  __host__ __device__ Layout(int C, int s_max, int nc) {
    Rcap = ceil_div(ceil_div(s_max, nc), kRowPad) * kRowPad;
    uint32_t off = 0;
    R = off;    off += 2u * Rcap * 128u;                 // [2 halves of D][Rcap][64] bf16, 128-byte swizzle
    P = off;    off += (uint32_t)C * 256u;               // prepared keys of the block; later the one-hot operand
    G = off;    off += (uint32_t)C * 256u;               // gated keys of the block
    xbuf = off; off += 2u * nc * C * 8u;                 // [parity][source CTA][token] {value, row}
    part = off; off += (2u * C * 8u > 4096u ? 2u * C * 8u : 4096u);                      // [column half][token] {value, row}: the two halves of a chunk (4 KB at least: see stat)
    tok = off;  off += 4u * C * 4u;                      // nov[C] f32, idx[C], pos[C], list[C]
    const uint32_t sp = (uint32_t)((s_max + 63) & ~31);  // padded row count: every region below stays 16-byte aligned
    rowi = off; off += sp * 4u + sp * 2u + ((2u * Rcap + 15u) & ~15u);  // cur[sp] i32, gci[sp] i16, lci[Rcap] i16 (by local row)
    tloc = off; off += ((2u * C + 15u) & ~15u) + 2u * sp;  // touched_local[C] u16, stamps[sp] u16 (update that last touched the row)
    stat = part;                                         // LayerNorm partial sums of the scatter epilogue (the routing partials are dead by then)
    bars = off; off += 448u;
    total = (off + 15u) & ~15u;
  }
};

struct Bars {
  uint64_t full_p, full_g;              // TMA arrivals of the block's prepared / gated keys
  // MMAs of a chunk complete, per tile of 128 tokens / ... and read back.  With at most 128 resident rows per CTA the
  // 256 accumulator columns of a token tile hold two chunks: consecutive passes alternate between the halves (first
  // index), so that a pass is issued while the workers still read the one before it
  uint64_t tm_full[2][2];
  uint64_t tm_empty[2][2];
  uint64_t w2i;                         // workers -> issuer: shared-memory operands are ready
  uint64_t sc_done;                     // scatter MMAs complete
  uint64_t xbar[2];                     // arrivals of the peers' partial results (two in flight)
  uint64_t zero_done;                   // the copy engine has cleared the one-hot operand
  uint32_t tmem_base;
  int abort;                            // somebody in the cluster gave up
  int n_pass;                           // scatter passes of the current update (workers -> issuer)
  float red_v[32];
  int red_t[32];
};

static_assert(kNewRows <= kWorkerWarps, "one warp per appended row in the short path");
static_assert(sizeof(Bars) <= 448, "the barrier block outgrew its shared-memory region");

struct Args {
  LayerDev L;
  const kvm_update_plan* plan;
  int n_plan;
  int nc;
  int s_max;             // final number of memory rows
  long long n_tok;       // tokens per kv row in pk_all / gk_all
  bf16* k_sum;           // [rows][capacity][D]
  bf16* k_attn;          // [rows][capacity][D] final view
  int capacity;
  bf16* pool_k;          // [rows][pool_rows][D] or null (no versions kept)
  long long pool_rows;
  int* ver_idx;          // [rows][ver_rows] or null
  long long ver_rows;
  int* route;            // [rows][n_plan][C]
  int* born;             // [rows][s_max] token that created each memory row, or null
  int* progress;         // [rows][nc] last update whose routes and version table are published (for the value-delta jobs
                         // that spare CTAs of this launch work on meanwhile), or null
  int* chain_done;       // CTAs of the routing that have finished
  int chain_ctas;        // CTAs of the routing (the CTAs behind them take value-delta jobs)
  int* status;
  uint32_t wait_limit;
  uint32_t test_flags;   // bit 0: the issuer withholds one commit (exercises the timeout path)
};

// Source of the copy that clears the one-hot operand of the scatter (64 KB of zeros, resident in L2).
__device__ __align__(128) unsigned char g_zeros[256 * 256];

// ------------------------------------------------------------------------------------------------ primitives
__device__ __forceinline__ void wsync() { asm volatile("bar.sync 1, %0;" ::"n"(kWorkers) : "memory"); }
// uniform AND over the worker threads
__device__ __forceinline__ bool wvote(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.and.pred q, 1, %2, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)ok), "n"(kWorkers)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ bool try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(tc::smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; also gives up when somebody else has.
template <bool CLUSTER = false>
__device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, uint32_t limit, volatile int* abort) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (CLUSTER ? try_wait_cluster(bar, parity) : tc::mbar_try_wait(bar, parity)) return true;
    if ((i & 63) == 63) {  // try_wait suspends the thread for a while by itself; look at the abort flag now and then
      if (*abort) return false;
      if (i >= 4096) __nanosleep(100);
    }
  }
  return false;
}
__device__ __forceinline__ uint32_t peer_addr(const void* local, int peer) {
  uint32_t a = tc::smem_u32(local), r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(peer));
  return r;
}
// 8-byte store into a peer's shared memory that completes 8 bytes of the transaction count of the peer's barrier:
// the data is visible to whoever has waited for that barrier phase (no fence, no separate arrival)
__device__ __forceinline__ void st_async_v2(uint32_t addr, float v, int i, uint32_t bar_addr) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];" ::"r"(addr),
               "r"(__float_as_uint(v)), "r"(i), "r"(bar_addr)
               : "memory");
}
__device__ __forceinline__ void st_peer_b32(uint32_t addr, int v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// 16-byte piece c (elements 8c..8c+7) of row r of an operand stored as [2 halves][rows][64] in the 128-byte swizzle
__device__ __forceinline__ uint32_t piece(int rows, int r, int c) {
  return (uint32_t)((c >> 3) * rows * 128 + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

// rows r < S owned by CTA `rank` (r % nc == rank)
__device__ __forceinline__ int n_local(int S, int nc, int rank) { return S > rank ? (S - rank + nc - 1) / nc : 0; }

// One thread: tiled TMA copies of block u of a kv row (prepared and gated keys, two 64-element halves each) into the
// block buffers.  The gated keys first: the logits pass, which opens an update, reads them.
__device__ __forceinline__ void issue_block_loads(unsigned char* smem, const Layout& lay, Bars* bars, const CUtensorMap* map_pk,
                                                  const CUtensorMap* map_gk, int row, long long n_tok, int C, int u) {
  const int y = (int)((long long)row * n_tok + (long long)u * C);
  tc::mbar_arrive_expect_tx(&bars->full_g, (uint32_t)C * 256u);
  tc::tma_load_2d(smem + lay.G, map_gk, 0, y, &bars->full_g);
  tc::tma_load_2d(smem + lay.G + C * 128, map_gk, 64, y, &bars->full_g);
  tc::mbar_arrive_expect_tx(&bars->full_p, (uint32_t)C * 256u);
  tc::tma_load_2d(smem + lay.P, map_pk, 0, y, &bars->full_p);
  tc::tma_load_2d(smem + lay.P + C * 128, map_pk, 64, y, &bars->full_p);
}

// ------------------------------------------------------------------------------------------------ the issuer
// One thread: TMA copies of the next block, the MMAs of the routing passes and of the scatter.
struct Issuer {
  const Args& a;
  unsigned char* smem;
  const Layout& lay;
  Bars* bars;
  uint32_t tmem;
  int crank, row;
  const CUtensorMap* map_pk;
  const CUtensorMap* map_gk;
  int which;             // 0: token tile 0, all copies, the scatter; 1: token tile 1 of the routing passes only
  uint32_t g = 0;        // chunks issued so far
  uint32_t n_w2i = 0, n_sc = 0, n_load = 0, n_zero = 0;
  volatile int* abort;
  // accumulator half and per-barrier phase of chunk number gg (see Bars::tm_full): with at most 128 resident rows per
  // CTA consecutive chunks alternate between the halves of a token tile's 256 columns
  __device__ __forceinline__ int acc_half(uint32_t gg) const { return lay.Rcap <= 128 ? (int)(gg & 1u) : 0; }
  __device__ __forceinline__ int acc_phase(uint32_t gg) const { return lay.Rcap <= 128 ? (int)(gg >> 1) : (int)gg; }

  // Update u of this CTA's rows is complete in global memory (routes, version table): tell the CTAs that work on the
  // value side.  Called behind a wait for all worker warps, whose writes this thread's fence makes visible with the flag.
  __device__ __forceinline__ void publish(int u) {
    if (a.progress == nullptr) return;
    __threadfence();
    *reinterpret_cast<volatile int*>(a.progress + (size_t)row * a.nc + crank) = u;
  }
  __device__ __forceinline__ bool wait_workers() {
    const bool ok = wait(&bars->w2i, n_w2i & 1, a.wait_limit, abort);
    ++n_w2i;
    tc::tc_fence_after_sync();
    return ok;
  }
  // warm L2 with a later block (the copy into shared memory then does not wait for DRAM)
  __device__ __forceinline__ void prefetch_block(int u) {
    const int C = a.L.C;
    const int y = (int)((long long)row * a.n_tok + (long long)u * C);
#pragma unroll
    for (int x = 0; x < 128; x += 64) {
      asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map_pk), "r"(x), "r"(y) : "memory");
      asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map_gk), "r"(x), "r"(y) : "memory");
    }
  }
  __device__ __forceinline__ void load_block(int u) { issue_block_loads(smem, lay, bars, map_pk, map_gk, row, a.n_tok, a.L.C, u); }
  // Operand descriptors and strides that never change, built once (the per-update code of this thread stays short: it
  // runs alone, so every instruction-cache line it touches for the first time in an update is a wait of its own).
  uint64_t d_p, d_g, d_r, d_new, d_gmn;  // prepared keys / one-hot (K-major), gated keys (K-major), resident rows, new rows, gated keys (MN-major)
  uint32_t a_half, r_half;               // second 64-element half of an operand, in descriptor units (16 bytes)
  __device__ __forceinline__ void setup() {
    const int C = a.L.C;
    d_p = tc::make_desc(tc::smem_u32(smem + lay.P), 16, 1024);
    d_g = tc::make_desc(tc::smem_u32(smem + lay.G), 16, 1024);
    d_r = tc::make_desc(tc::smem_u32(smem + lay.R), 16, 1024);
    d_new = tc::make_desc(tc::smem_u32(smem + lay.part), 16, 1024);
    d_gmn = tc::make_desc(tc::smem_u32(smem + lay.G), (uint32_t)C * 128u, 1024);
    a_half = (uint32_t)(C * 128) >> 4;
    r_half = (uint32_t)(lay.Rcap * 128) >> 4;
  }
  // S[tokens x rows] = A[tokens x D] * R[rows x D]^T over the first n_rows local rows, up to 256 rows per chunk: one
  // MMA per token tile and k-step covers the whole chunk (issuing an MMA costs about as much as executing a small
  // one), the accumulators of token tile m live in tensor-memory columns [256 m, 256 m + N).  One commit per token
  // tile, so that the first tile is read back while the second is computed.  The loops are kept rolled on purpose.
  __device__ __forceinline__ bool pass(uint64_t da_base, int n_rows, bool withhold_first_commit) {
    const int n_mt = a.L.C / 128;
    const int n_chunks = ceil_div(n_rows, kChunk);
    for (int c = 0; c < n_chunks; ++c, ++g) {
      const int n = min(kChunk, n_rows - c * kChunk);
      const uint32_t idesc = tc::make_idesc(128, (n + 15) & ~15, 0, 0);
      const uint64_t db0 = d_r + (uint64_t)((uint32_t)(c * kChunk * 128) >> 4);
      for (int m = which; m < n_mt; m += kIssuers) {
        const int hb = acc_half(g), ph = acc_phase(g);
        if (ph >= 1 && !wait(&bars->tm_empty[hb][m], (ph - 1) & 1, a.wait_limit, abort)) return false;
        tc::tc_fence_after_sync();
        const uint64_t da0 = da_base + (uint64_t)((uint32_t)(m * 128 * 128) >> 4);
        const uint32_t d = tmem + (uint32_t)(m * kChunk + hb * 128);
#pragma unroll 1
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t lo = (uint32_t)(ks & 3) * 2u;
          tc::mma_ss(d, da0 + (uint64_t)(((ks >> 2) ? a_half : 0u) + lo), db0 + (uint64_t)(((ks >> 2) ? r_half : 0u) + lo), idesc, ks > 0);
        }
        if (!(withhold_first_commit && c == 0 && m == 0)) tc::mma_commit_own_cta(&bars->tm_full[hb][m]);
      }
    }
    return true;
  }
  // Logits of every token against the rows that were just appended (at most kNewRows of them), which every CTA keeps
  // as a small operand of its own: S[tokens x 16] = gk[tokens x D] * newk[16 x D]^T
  __device__ __forceinline__ bool pass_new_rows() {
    const int n_mt = a.L.C / 128;
    constexpr uint32_t idesc = tc::make_idesc(128, kNewRows, 0, 0);
    constexpr uint32_t n_half = (uint32_t)(kNewRows * 128) >> 4;
    for (int m = which; m < n_mt; m += kIssuers) {
      const int hb = acc_half(g), ph = acc_phase(g);
      if (ph >= 1 && !wait(&bars->tm_empty[hb][m], (ph - 1) & 1, a.wait_limit, abort)) return false;
      tc::tc_fence_after_sync();
      const uint64_t da0 = d_g + (uint64_t)((uint32_t)(m * 128 * 128) >> 4);
      const uint32_t d = tmem + (uint32_t)(m * kChunk + hb * 128);
#pragma unroll 1
      for (int ks = 0; ks < HD / 16; ++ks) {
        const uint32_t lo = (uint32_t)(ks & 3) * 2u;
        tc::mma_ss(d, da0 + (uint64_t)(((ks >> 2) ? a_half : 0u) + lo), d_new + (uint64_t)(((ks >> 2) ? n_half : 0u) + lo), idesc, ks > 0);
      }
      tc::mma_commit_own_cta(&bars->tm_full[hb][m]);
    }
    ++g;
    return true;
  }
  // delta[128 compacted rows x D] = onehot[rows x C tokens] * gk[C tokens x D]
  // (one-hot: K-major [C/64][128][64] in the buffer of the prepared keys; gated keys: MN-major)
  __device__ __forceinline__ void scatter() {
    constexpr uint32_t idesc = tc::make_idesc(128, HD, 0, 1);
    const int n_ks = a.L.C / 16;
#pragma unroll 1
    for (int ks = 0; ks < n_ks; ++ks)
      tc::mma_ss(tmem, d_p + (uint64_t)((uint32_t)(ks >> 2) * (128u * 128u >> 4) + (uint32_t)(ks & 3) * 2u), d_gmn + (uint64_t)((uint32_t)ks * (2048u >> 4)), idesc, ks > 0);
    tc::mma_commit_own_cta(&bars->sc_done);
  }

  __device__ bool run() {
    const int C = a.L.C, nc = a.nc;
    // The second issuer follows the same schedule and takes part in the same handshakes, but only issues the routing
    // MMAs of its token tile.
    const bool primary = which == 0;
    setup();
    // block 0 (the initial memory) needs the prepared keys only; the gated keys travel with it to keep the barriers in step
    if (primary) load_block(0);
    kvm_update_plan pl_next = a.plan[0];  // fetched one update ahead: the table lives in global memory
    for (int u = 0; u < a.n_plan; ++u) {
      const kvm_update_plan pl = pl_next;
      if (u + 1 < a.n_plan) pl_next = a.plan[u + 1];
      const int S0 = pl.state_before, na = pl.n_append, S1 = S0 + na, nm = C - na;
      if (u == 0) {
        // the workers build the initial memory from the prepared keys and report when the block buffers are free
        if (!wait_workers()) return false;
        if (primary) publish(0);
        n_load = 1;
        if (primary && a.n_plan > 1) load_block(1);
        if (primary && a.n_plan > 2 && crank == 0) prefetch_block(2);
        continue;
      }
      const bool has_nov = na > 0 && nm > 0;
      if (primary && u + 2 < a.n_plan && crank == (u & (nc - 1))) prefetch_block(u + 2);  // one CTA of the cluster asks, all profit
      const bool withhold = (a.test_flags & 1u) && u == 1;
      if (nm > 0 && na <= kNewRows) {
        // few appended rows: the logits against the OLD memory do not depend on them, so they go first and the
        // novelty MMAs follow behind (the workers read one result while the tensor core produces the next); the
        // logits against the new rows are a small third pass once the workers have chosen and stored them
        if (!wait(&bars->full_g, n_load & 1, a.wait_limit, abort)) return false;
        if (!pass(d_g, n_local(S0, nc, crank), withhold)) return false;
        if (has_nov) {
          if (!wait(&bars->full_p, n_load & 1, a.wait_limit, abort)) return false;
          if (!pass(d_p, n_local(S0, nc, crank), false)) return false;
        }
        // The workers report when nobody reads the prepared keys any more (novelty read back, appended rows stored, the
        // new rows in every CTA's small operand): the copy engine clears their buffer, which becomes the one-hot operand
        // of the scatter, while the workers score the new rows and build the routing table.
        if (!wait_workers()) return false;
        if (primary) {
          // (an update without appends never looked at the prepared keys: their copy must have landed before the buffer is reused)
          if (!has_nov && !wait(&bars->full_p, n_load & 1, a.wait_limit, abort)) return false;
          tc::mbar_arrive_expect_tx(&bars->zero_done, (uint32_t)C * 256u);
          tc::bulk_g2s(smem + lay.P, g_zeros, (uint32_t)C * 256u, &bars->zero_done);
        }
        if (has_nov && na > kDirectNew && !pass_new_rows()) return false;  // (one or two new rows are scored by the workers with plain dot products)
      } else {
        if (has_nov) {
          if (!wait(&bars->full_p, n_load & 1, a.wait_limit, abort)) return false;
          if (!pass(d_p, n_local(S0, nc, crank), false)) return false;
          if (!wait_workers()) return false;  // the appended rows are in the resident memory
        }
        if (nm > 0) {
          if (!wait(&bars->full_g, n_load & 1, a.wait_limit, abort)) return false;
          if (!pass(d_g, n_local(S1, nc, crank), withhold)) return false;
        }
      }
      // scatter passes (their number is decided by the workers once the routing is final)
      if (!wait_workers()) return false;
      const int n_pass = *reinterpret_cast<volatile int*>(&bars->n_pass);
      for (int p = 0; p < n_pass; ++p) {
        if (p > 0 && !wait_workers()) return false;
        if (primary) scatter();
        ++n_sc;
      }
      if (n_pass == 0) {  // nothing routed to this CTA's rows: the logits MMAs must still be complete before G is overwritten
        if (primary) tc::mma_commit_own_cta(&bars->sc_done);
        ++n_sc;
      }
      // (all routing MMAs were read back by the workers before they asked for the scatter, so the commit of the
      // primary issuer covers what the block buffers are needed for)
      if (primary && !wait(&bars->sc_done, (n_sc - 1) & 1, a.wait_limit, abort)) return false;
      if (nm > 0 && na <= kNewRows) {  // the clearing copy has landed, too (nobody may have waited for it: no row of this CTA touched)
        if (primary && !wait(&bars->zero_done, n_zero & 1, a.wait_limit, abort)) return false;
        ++n_zero;
      }
      ++n_load;  // the loads of this update have been consumed; a worker thread has issued the next block's (see there)
      // the next routing pass reads the resident memory the workers are refreshing now
      if (!wait_workers()) return false;
      if (primary) publish(u);
    }
    return true;
  }
};

// ------------------------------------------------------------------------------------------------ the workers
struct Workers {
  const Args& a;
  unsigned char* smem;
  const Layout& lay;
  Bars* bars;
  uint32_t tmem;
  int crank, row;
  const float* ln_w;
  const float* ln_b;
  volatile int* abort;
  int tid, warp, lane;
  const CUtensorMap* map_pk;
  const CUtensorMap* map_gk;
  uint32_t g = 0, n_sc = 0, n_x = 0, n_load = 0, n_zero = 0;
  int pool_next = 0;
  unsigned mine_mask = 0;  // lanes whose row (a multiple of 32 + lane) belongs to this CTA
  // accumulator half and per-barrier phase of chunk number gg (see Bars::tm_full): with at most 128 resident rows per
  // CTA consecutive chunks alternate between the halves of a token tile's 256 columns
  __device__ __forceinline__ int acc_half(uint32_t gg) const { return lay.Rcap <= 128 ? (int)(gg & 1u) : 0; }
  __device__ __forceinline__ int acc_phase(uint32_t gg) const { return lay.Rcap <= 128 ? (int)(gg >> 1) : (int)gg; }

  __device__ __forceinline__ float* nov() const { return reinterpret_cast<float*>(smem + lay.tok); }
  __device__ __forceinline__ int* idx() const { return reinterpret_cast<int*>(smem + lay.tok) + a.L.C; }
  __device__ __forceinline__ int* pos() const { return reinterpret_cast<int*>(smem + lay.tok) + 2 * a.L.C; }
  __device__ __forceinline__ int* list() const { return reinterpret_cast<int*>(smem + lay.tok) + 3 * a.L.C; }
  __device__ __forceinline__ int* cur() const { return reinterpret_cast<int*>(smem + lay.rowi); }
  __device__ __forceinline__ int padded_rows() const { return (a.s_max + 63) & ~31; }
  __device__ __forceinline__ short* gci() const { return reinterpret_cast<short*>(smem + lay.rowi + (uint32_t)padded_rows() * 4u); }
  __device__ __forceinline__ short* lci() const { return gci() + padded_rows(); }  // indexed by the local row r / nc
  __device__ __forceinline__ unsigned short* tloc() const { return reinterpret_cast<unsigned short*>(smem + lay.tloc); }
  __device__ __forceinline__ unsigned short* tf() const { return reinterpret_cast<unsigned short*>(smem + lay.tloc + ((2u * a.L.C + 15u) & ~15u)); }
  __device__ __forceinline__ float2* part(int half) const { return reinterpret_cast<float2*>(smem + lay.part) + half * a.L.C; }
  __device__ __forceinline__ float2* xb(int parity, int src) const { return reinterpret_cast<float2*>(smem + lay.xbuf) + (size_t)(parity * a.nc + src) * a.L.C; }
  __device__ __forceinline__ float* stat(int which) const { return reinterpret_cast<float*>(smem + lay.stat) + which * 4 * 128; }

  __device__ __forceinline__ void signal_issuer() {
    tc::fence_proxy_async();   // shared-memory writes of this thread -> visible to the tensor core / TMA
    tc::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&bars->w2i);
  }

  // Read back the chunks of a routing pass.  ARG = false: running maximum (novelty); true: running first-argmax of
  // rows >= `protected_rows`.  Warp w reads token tile (w / 4) % 2, lanes 32 (w % 4).., and one half of the chunk's
  // 32-column groups; leaves per token the CTA's partial result in part(half)[token].
  template <bool ARG>
  __device__ __forceinline__ bool read_pass(int n_rows, int protected_rows) {
    float v;
    int i;
    const bool ok = read_regs<ARG>(n_rows, protected_rows, v, i);
    const int half = warp >> 3, mt = (warp >> 2) & 1, quarter = warp & 3;
    if (mt * 128 < a.L.C) part(half)[mt * 128 + quarter * 32 + lane] = make_float2(v, __int_as_float(i));
    return wvote(ok);
  }
  // The same, the thread's result (value; global row or -1) left in registers, no vote.
  template <bool ARG>
  __device__ __forceinline__ bool read_regs(int n_rows, int protected_rows, float& v_out, int& i_out) {
    const int C = a.L.C, nc = a.nc;
    const int half = warp >> 3, mt = (warp >> 2) & 1, quarter = warp & 3;
    const bool active = mt * 128 < C;
    const int n_chunks = ceil_div(n_rows, kChunk);
    // first local row that counts: global row l * nc + crank >= protected_rows
    const int l_min = ARG ? (protected_rows > crank ? (protected_rows - crank + nc - 1) / nc : 0) : 0;
    float bv[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    int bi[4] = {-1, -1, -1, -1};
    bool ok = true;
    for (int c = 0; c < n_chunks; ++c, ++g) {
      if (!active) continue;
      const int hb = acc_half(g), ph = acc_phase(g);
      ok = ok && wait(&bars->tm_full[hb][mt], ph & 1, a.wait_limit, abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;  // the caller aborts
      tc::tc_fence_after_sync();
      const int n = min(kChunk, n_rows - c * kChunk);
      const int n_groups = ceil_div(n, 32), g_half = (n_groups + 1) / 2;
      const int g_begin = half ? g_half : 0, g_end = half ? n_groups : g_half;
      for (int gi = g_begin; gi < g_end; ++gi) {
        uint32_t r[32];
        tc::tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * kChunk + hb * 128 + gi * 32), r);
        tc::tmem_ld_wait();
        const int l0 = c * kChunk + gi * 32;  // local row of column 0
        const bool full = l0 + 32 <= n_rows && l0 >= l_min;
        if (!ARG) {
          if (full) {
#pragma unroll
            for (int j = 0; j < 32; ++j) bv[j & 3] = fmaxf(bv[j & 3], __uint_as_float(r[j]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (l0 + j < n_rows) bv[j & 3] = fmaxf(bv[j & 3], __uint_as_float(r[j]));
          }
        } else {
          if (full) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float x = __uint_as_float(r[j]);  // strictly greater replaces: the first of equal values stays
              if (x > bv[j & 3]) { bv[j & 3] = x; bi[j & 3] = l0 + j; }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float x = __uint_as_float(r[j]);
              const int l = l0 + j;
              if (l < n_rows && l >= l_min && x > bv[j & 3]) { bv[j & 3] = x; bi[j & 3] = l; }
            }
          }
        }
      }
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&bars->tm_empty[hb][mt]);
    }
    float v = bv[0];
    int i = bi[0];
    if (!ARG) {
      v = fmaxf(fmaxf(bv[0], bv[1]), fmaxf(bv[2], bv[3]));
    } else {
#pragma unroll
      for (int j = 1; j < 4; ++j)  // first maximum in row order: larger value, or equal value at a lower row
        if (bi[j] >= 0 && (i < 0 || bv[j] > v || (bv[j] == v && bi[j] < i))) { v = bv[j]; i = bi[j]; }
      if (i >= 0) i = i * nc + crank;  // local -> global row
    }
    v_out = v;
    i_out = i;
    return ok;
  }

  // Merge the two column halves, exchange the CTA's partial results with the peers, combine.
  // ARG = false: nov()[t] = bf16(max); true: idx()[t] = first row with the largest logit.
  template <bool ARG>
  __device__ __forceinline__ bool exchange() {
    const int C = a.L.C, nc = a.nc;
    const int parity = n_x & 1;
    float v = -INFINITY;
    int i = -1;
    if (tid < C) {
      const float2 p0 = part(0)[tid], p1 = part(1)[tid];
      v = p0.x;
      i = __float_as_int(p0.y);
      const int i1 = __float_as_int(p1.y);
      if (!ARG) {
        v = fmaxf(p0.x, p1.x);
      } else if (i1 >= 0 && (i < 0 || p1.x > v || (p1.x == v && i1 < i))) {
        v = p1.x;
        i = i1;
      }
    }
    bool ok = true;
    if (nc > 1) {
      // every token's partial result goes to the same token's slot in every peer; this CTA expects the peers' bytes
      if (tid == 0) tc::mbar_arrive_expect_tx(&bars->xbar[parity], (uint32_t)((nc - 1) * C * 8));
      if (tid < C) {
        const float2* slot = &xb(parity, crank)[tid];
        for (int p = 0; p < nc; ++p)
          if (p != crank) st_async_v2(peer_addr(slot, p), v, i, peer_addr(&bars->xbar[parity], p));
      }
      ok = tid < C ? wait<true>(&bars->xbar[parity], (n_x >> 1) & 1, a.wait_limit, abort) : true;
      if (ok && tid < C) {
        for (int p = 0; p < nc; ++p) {
          if (p == crank) continue;
          const float2 q = xb(parity, p)[tid];
          const int qi = __float_as_int(q.y);
          if (!ARG) v = fmaxf(v, q.x);
          else if (qi >= 0 && (i < 0 || q.x > v || (q.x == v && qi < i))) { v = q.x; i = qi; }
        }
      }
    }
    ++n_x;
    if (tid < C) {
      if (!ARG) nov()[tid] = bf16_round(v);
      else idx()[tid] = i;
    }
    return wvote(ok);
  }

  // Both routing results of the logits-first order in one exchange.  part(half)[token] holds {best logit over the
  // old rows, row (16 bits, 0xffff = none) | novelty maximum as bf16 << 16}; the bf16 rounding of the novelty commutes
  // with the maximum.  Leaves the novelty in nov()[token] and the best old row in the token thread's registers.
  __device__ __forceinline__ bool exchange_both(float& best_v, int& best_i) {
    const int C = a.L.C, nc = a.nc;
    const int parity = n_x & 1;
    float v = -INFINITY, nv = -INFINITY;
    int i = -1;
    auto take = [&](float2 p) {
      const unsigned w = __float_as_uint(p.y);
      const int pi = (w & 0xffffu) == 0xffffu ? -1 : (int)(w & 0xffffu);
      nv = fmaxf(nv, __uint_as_float(w & 0xffff0000u));
      if (pi >= 0 && (i < 0 || p.x > v || (p.x == v && pi < i))) { v = p.x; i = pi; }
    };
    if (tid < C) {
      take(part(0)[tid]);
      take(part(1)[tid]);
    }
    bool ok = true;
    if (nc > 1) {
      if (tid == 0) tc::mbar_arrive_expect_tx(&bars->xbar[parity], (uint32_t)((nc - 1) * C * 8));
      if (tid < C) {
        const float2* slot = &xb(parity, crank)[tid];
        const int packed = (int)(((unsigned)i & 0xffffu) | (__float_as_uint(nv) & 0xffff0000u));
        for (int p = 0; p < nc; ++p)
          if (p != crank) st_async_v2(peer_addr(slot, p), v, packed, peer_addr(&bars->xbar[parity], p));
      }
      ok = tid < C ? wait<true>(&bars->xbar[parity], (n_x >> 1) & 1, a.wait_limit, abort) : true;
      if (ok && tid < C)
        for (int p = 0; p < nc; ++p)
          if (p != crank) take(xb(parity, p)[tid]);
    }
    ++n_x;
    if (tid < C) nov()[tid] = nv;
    best_v = v;
    best_i = i;
    return wvote(ok);
  }

  // LayerNorm view of one memory row (8 lanes per row): source `x`, written to the resident memory (if local) and
  // to a pool row / the carried sums.
  // `new_row` >= 0: also row `new_row` of the small operand every CTA keeps of the rows appended in this update.
  __device__ __forceinline__ void store_key_row(RowVec<HD, 8>& x, int r, int slot, int gl, bool mine, int new_row = -1) {
    const size_t grow = (size_t)row * a.capacity + r;
    if (mine) store_row<HD, 8>(x, a.k_sum + grow * HD, gl);
    layer_norm_row<HD, 8>(x, ln_w, ln_b, a.L.ln_eps, gl);
    uint4 u0, u1;
    u0.x = pack_bf16(x.x[0], x.x[1]); u0.y = pack_bf16(x.x[2], x.x[3]); u0.z = pack_bf16(x.x[4], x.x[5]); u0.w = pack_bf16(x.x[6], x.x[7]);
    u1.x = pack_bf16(x.x[8], x.x[9]); u1.y = pack_bf16(x.x[10], x.x[11]); u1.z = pack_bf16(x.x[12], x.x[13]); u1.w = pack_bf16(x.x[14], x.x[15]);
    if (new_row >= 0) {
      *reinterpret_cast<uint4*>(smem + lay.part + piece(kNewRows, new_row, 2 * gl)) = u0;
      *reinterpret_cast<uint4*>(smem + lay.part + piece(kNewRows, new_row, 2 * gl + 1)) = u1;
    }
    if (mine) {
      const int l = r / a.nc;
      *reinterpret_cast<uint4*>(smem + lay.R + piece(lay.Rcap, l, 2 * gl)) = u0;
      *reinterpret_cast<uint4*>(smem + lay.R + piece(lay.Rcap, l, 2 * gl + 1)) = u1;
      if (a.pool_k) {
        bf16* dst = a.pool_k + ((size_t)row * a.pool_rows + slot) * HD + gl * 16;
        *reinterpret_cast<uint4*>(dst) = u0;
        *reinterpret_cast<uint4*>(dst + 8) = u1;
      }
    }
  }
  // the 16 elements of lane gl of row t of a block operand (prepared or gated keys)
  __device__ __forceinline__ void load_block_row(RowVec<HD, 8>& x, uint32_t off, int t, int gl) { load_block_row_n(x, off, a.L.C, t, gl); }
  // ... of an operand of `rows` rows
  __device__ __forceinline__ void load_block_row_n(RowVec<HD, 8>& x, uint32_t off, int rows, int t, int gl) {
    const int C = rows;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint4 u = *reinterpret_cast<const uint4*>(smem + off + piece(C, t, 2 * gl + h));
      const float2 p0 = unpack_bf16(u.x), p1 = unpack_bf16(u.y), p2 = unpack_bf16(u.z), p3 = unpack_bf16(u.w);
      x.x[h * 8 + 0] = p0.x; x.x[h * 8 + 1] = p0.y; x.x[h * 8 + 2] = p1.x; x.x[h * 8 + 3] = p1.y;
      x.x[h * 8 + 4] = p2.x; x.x[h * 8 + 5] = p2.y; x.x[h * 8 + 6] = p3.x; x.x[h * 8 + 7] = p3.y;
    }
  }

  // rows [S0, S0 + na) from the tokens list()[0..na): `src_off` = operand holding what is stored (prepared or gated keys)
  // `all_ctas`: every CTA also keeps the rows' view in its small operand of new rows (na <= kNewRows)
  __device__ __forceinline__ void append_rows(int S0, int na, uint32_t src_off, int u, bool all_ctas = false) {
    const int gl = tid & 7, grp = tid >> 3;
    for (int base = 0; base < na; base += kWorkers / 8) {  // whole warps stay together: the LayerNorm uses group shuffles
      const int p = base + grp;
      const bool act = p < na;
      if (!__any_sync(0xffffffffu, act && (all_ctas || (S0 + p) % a.nc == crank))) continue;  // nothing for this warp to store
      const int r = S0 + (act ? p : 0);
      const int t = list()[act ? p : 0];
      RowVec<HD, 8> x;
      load_block_row(x, src_off, t, gl);
      const bool mine = act && (r % a.nc == crank);
      store_key_row(x, r, pool_next + p, gl, mine, (all_ctas && act) ? p : -1);
      if (mine && gl == 0 && a.born) a.born[(size_t)row * a.s_max + r] = u * a.L.C + t;
    }
    for (int i = tid; i < na; i += kWorkers) cur()[S0 + i] = pool_next + i;
    pool_next += na;
  }

  // The same for at most kWorkerWarps rows, one warp per row and four elements per lane, every CTA keeping the rows' view
  // in its small operand of new rows: the few warps that store rows run alone, and what they wait for is mostly their
  // own instructions, so the code is kept short.
  __device__ __forceinline__ void append_rows_warp(int S0, int na, uint32_t src_off, int u) {
    if (warp < na) {
      const int p = warp, r = S0 + p, t = list()[p], pc = lane >> 1;
      const uint32_t sub = (uint32_t)(lane & 1) * 8u;  // which half of a 16-byte piece
      const uint2 raw = *reinterpret_cast<const uint2*>(smem + src_off + piece(a.L.C, t, pc) + sub);
      RowVec<HD, 32> x;
      const float2 e0 = unpack_bf16(raw.x), e1 = unpack_bf16(raw.y);
      x.x[0] = e0.x; x.x[1] = e0.y; x.x[2] = e1.x; x.x[3] = e1.y;
      const bool mine = r % a.nc == crank;
      if (mine) *reinterpret_cast<uint2*>(a.k_sum + ((size_t)row * a.capacity + r) * HD + lane * 4) = raw;  // the carried sum is the token's row
      layer_norm_row<HD, 32>(x, ln_w, ln_b, a.L.ln_eps, lane);
      uint2 o;
      o.x = pack_bf16(x.x[0], x.x[1]);
      o.y = pack_bf16(x.x[2], x.x[3]);
      *reinterpret_cast<uint2*>(smem + lay.part + piece(kNewRows, p, pc) + sub) = o;
      if (mine) {
        *reinterpret_cast<uint2*>(smem + lay.R + piece(lay.Rcap, r / a.nc, pc) + sub) = o;
        if (a.pool_k) *reinterpret_cast<uint2*>(a.pool_k + ((size_t)row * a.pool_rows + pool_next + p) * HD + lane * 4) = o;
        if (lane == 0 && a.born) a.born[(size_t)row * a.s_max + r] = u * a.L.C + t;
      }
    }
    if (tid < na) cur()[S0 + tid] = pool_next + tid;
    pool_next += na;
  }

  __device__ bool run() {
    const int C = a.L.C, nc = a.nc;
    for (int l = crank; l < 32; l += nc) mine_mask |= 1u << l;
    int* route_row = a.route + (size_t)row * a.n_plan * C;
    kvm_update_plan pl_next = a.plan[0];  // fetched one update ahead
    for (int u = 0; u < a.n_plan; ++u) {
      const kvm_update_plan pl = pl_next;
      if (u + 1 < a.n_plan) pl_next = a.plan[u + 1];
      const int S0 = pl.state_before, na = pl.n_append, S1 = S0 + na, nm = C - na;
      int* ver = (a.ver_idx && pl.version_row >= 0) ? a.ver_idx + (size_t)row * a.ver_rows + pl.version_row : nullptr;
      bool ok = true;
      if (u == 0) {
        // ---- initial memory: the first C tokens row for row (model/kvm_mixer.py:434-447)
        ok = wait(&bars->full_p, 0, a.wait_limit, abort) && wait(&bars->full_g, 0, a.wait_limit, abort);
        if (!wvote(ok)) return false;
        if (tid < C) list()[tid] = tid;
        wsync();
        append_rows(0, na, (a.L.gate_initial && a.L.gate_keys) ? lay.G : lay.P, 0);
        if (crank == 0)
          for (int i = tid; i < C; i += kWorkers) route_row[i] = i < na ? -(1 + i) : 0;
        wsync();
        if (ver)
          for (int i = tid + crank * kWorkers; i < S1; i += kWorkers * nc) ver[i] = cur()[i];
        n_load = 1;
        signal_issuer();
        continue;
      }
      const bool has_nov = na > 0 && nm > 0;
      const int protected_rows = min(a.L.sink_len, S1);
      // few appended rows: logits against the old memory first, the novelty behind them, both exchanged together,
      // the logits against the new rows last (see the issuer)
      const bool fast = nm > 0 && na <= kNewRows;
      float best_v = -INFINITY;  // (fast) this token's best logit and row so far
      int best_i = -1;
      // ---- 1. novelty of every token against the old memory; the n_append least similar tokens are appended
      if (fast) {
        float vl_, vn_ = -INFINITY;
        int il_, unused;
        bool okr = read_regs<true>(n_local(S0, nc, crank), protected_rows, vl_, il_);
        if (has_nov) okr = read_regs<false>(n_local(S0, nc, crank), 0, vn_, unused) && okr;
        const int mt = (warp >> 2) & 1;
        if (mt * 128 < C) {
          const unsigned packed = ((unsigned)il_ & 0xffffu) | ((unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(vn_)) << 16);
          part(warp >> 3)[mt * 128 + (warp & 3) * 32 + lane] = make_float2(vl_, __uint_as_float(packed));
        }
        if (!wvote(okr)) return false;
        if (!exchange_both(best_v, best_i)) return false;
      } else if (has_nov) {
        if (!read_pass<false>(n_local(S0, nc, crank), 0)) return false;
        if (!exchange<false>()) return false;
      }
      if (na > 0) {
        if (!has_nov) {  // the whole block is appended
          ok = wait(&bars->full_p, n_load & 1, a.wait_limit, abort);
          if (!wvote(ok)) return false;
          if (tid < C) { pos()[tid] = tid; list()[tid] = tid; idx()[tid] = -1; }
        } else if (na == 1) {
          // the token with the lowest novelty, lowest index among equals
          float bv = tid < C ? nov()[tid] : INFINITY;
          int bt = tid < C ? tid : 0x7fffffff;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int ot = __shfl_xor_sync(0xffffffffu, bt, off);
            if (ov < bv || (ov == bv && ot < bt)) { bv = ov; bt = ot; }
          }
          if (lane == 0) { bars->red_v[warp] = bv; bars->red_t[warp] = bt; }
          wsync();
          bv = bars->red_v[lane & 15];
          bt = bars->red_t[lane & 15];
#pragma unroll
          for (int off = 8; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int ot = __shfl_xor_sync(0xffffffffu, bt, off);
            if (ov < bv || (ov == bv && ot < bt)) { bv = ov; bt = ot; }
          }
          if (tid < C) pos()[tid] = tid == bt ? 0 : -1;
          if (tid == 0) list()[0] = bt;
        } else {
          // stable rank of the novelty scores: the na lowest are appended, in token order
          int f = 0;
          if (tid < C) {
            const float si = nov()[tid];
            int rank = 0;
#pragma unroll 4
            for (int u0 = 0; u0 < C; u0 += 4) {
              const float4 q = *reinterpret_cast<const float4*>(nov() + u0);
              rank += (q.x < si || (q.x == si && u0 + 0 < tid)) ? 1 : 0;
              rank += (q.y < si || (q.y == si && u0 + 1 < tid)) ? 1 : 0;
              rank += (q.z < si || (q.z == si && u0 + 2 < tid)) ? 1 : 0;
              rank += (q.w < si || (q.w == si && u0 + 3 < tid)) ? 1 : 0;
            }
            f = rank < na ? 1 : 0;
          }
          const unsigned bal = __ballot_sync(0xffffffffu, f != 0);
          if (lane == 0) bars->red_t[warp] = __popc(bal);
          wsync();
          if (tid < C) {
            int p = __popc(bal & ((1u << lane) - 1u));
            for (int w = 0; w < warp; ++w) p += bars->red_t[w];
            pos()[tid] = f ? p : -1;
            if (f) list()[p] = tid;
          }
        }
        wsync();
        if (fast) append_rows_warp(S0, na, (a.L.gate_appends && a.L.gate_keys) ? lay.G : lay.P, u);
        else append_rows(S0, na, (a.L.gate_appends && a.L.gate_keys) ? lay.G : lay.P, u);
        if (!fast && has_nov) signal_issuer();  // the appended rows are in place: the pass against them may start
      } else if (tid < C) {
        pos()[tid] = -1;
      }
      // The prepared keys are dead from here on: their buffer becomes the one-hot operand of the scatter.
      if (fast) {
        signal_issuer();  // the issuer has the copy engine clear it (and may start the pass against the new rows)
      } else if (nm > 0) {
        wsync();  // the warps that store appended rows have read their prepared keys
        uint4* o = reinterpret_cast<uint4*>(smem + lay.P);
        for (int i = tid; i < C * 16; i += kWorkers) o[i] = make_uint4(0, 0, 0, 0);  // while the tensor core works on the logits
      }
      // ---- 2. merge target of every token: first argmax of the fp32 logits over the memory after the appends
      if (fast) {
        bool okm = true;
        if (na > 0 && na <= kDirectNew) {
          // one or two new rows: fp32 dot products of every token's gated key with them, eight lanes per token (fixed
          // summation order); the rows are read from the small operand every CTA keeps of them
          // (results in the novelty and append-list arrays, which nobody reads any more in this update)
          wsync();  // the new rows are in the small operand (stored by the warps that appended them)
          float* dots_row[2] = {nov(), reinterpret_cast<float*>(list())};
          static_assert(kDirectNew <= 2, "two scratch rows");
          const int gl = tid & 7, grp = tid >> 3;
          for (int j = 0; j < na; ++j) {
            RowVec<HD, 8> nr;
            load_block_row_n(nr, lay.part, kNewRows, j, gl);
            for (int base = 0; base < C; base += kWorkers / 8) {
              const int t = base + grp;
              RowVec<HD, 8> kr;
              load_block_row(kr, lay.G, t, gl);
              float acc = 0.f;
#pragma unroll
              for (int e = 0; e < HD / 8; ++e) acc = fmaf(kr.x[e], nr.x[e], acc);
              acc = group_sum<8>(acc);
              if (gl == 0) dots_row[j][t] = acc;
            }
          }
          wsync();
          if (tid < C)
            for (int j = 0; j < na; ++j) {
              const float x = dots_row[j][tid];
              if (S0 + j >= protected_rows && (x > best_v || best_i < 0)) { best_v = x; best_i = S0 + j; }
            }
        } else if (na > 0) {
          // the new rows (columns 0 .. na-1 of the small pass) against this token's best old row: a new row has the
          // higher index, it wins only with a strictly larger logit
          const int mt = (warp >> 2) & 1;
          if (mt * 128 < C) {
            const int hb = acc_half(g), ph = acc_phase(g);
            okm = wait(&bars->tm_full[hb][mt], ph & 1, a.wait_limit, abort);
            okm = __all_sync(0xffffffffu, okm);
            if (okm && warp * 32 < C) {
              tc::tc_fence_after_sync();
              uint32_t r16[16];
              tc::tmem_ld16(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(mt * kChunk + hb * 128), r16);
              tc::tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < kNewRows; ++j) {
                const float x = __uint_as_float(r16[j]);
                if (j < na && S0 + j >= protected_rows && (x > best_v || best_i < 0)) { best_v = x; best_i = S0 + j; }
              }
              tc::tc_fence_before_sync();
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&bars->tm_empty[hb][mt]);
          }
          ++g;
        }
        if (tid < C) idx()[tid] = best_i;
        if (!wvote(okm)) return false;
      } else if (nm > 0) {
        if (!read_pass<true>(n_local(S1, nc, crank), protected_rows)) return false;
        if (!exchange<true>()) return false;
      }
      // ---- 3. routing table, touched rows and their pool slots
      int my = -1;
      if (tid < C) {
        const int p = pos()[tid];
        my = p >= 0 ? -1 : idx()[tid];
        if (crank == 0) route_row[(size_t)u * C + tid] = p >= 0 ? -(1 + S0 + p) : my;
      }
      // a row is touched in this update iff its stamp equals the update's number (no clearing between updates)
      if (my >= 0) tf()[my] = (unsigned short)u;
      wsync();
      int n_touched = 0, n_touched_local = 0;
      {
        // compact index of every touched row among all touched rows (pool slot) and among this CTA's (accumulator lane)
        int base_all = 0, base_loc = 0;
        for (int r0 = 0; r0 < S1; r0 += kWorkers) {
          const int r = r0 + tid;
          const bool t = r < S1 && tf()[r] == (unsigned short)u;
          const unsigned bal = __ballot_sync(0xffffffffu, t);
          if (lane == 0) {
            bars->red_t[warp] = __popc(bal);
            bars->red_t[16 + warp] = __popc(bal & mine_mask);
          }
          wsync();
          // lanes 0..15 hold the counts of all rows, lanes 16..31 of this CTA's rows: inclusive scan over each half
          int cnt = bars->red_t[lane];
#pragma unroll
          for (int d = 1; d < 16; d <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, cnt, d, 16);
            if ((lane & 15) >= d) cnt += y;
          }
          const int ta = __shfl_sync(0xffffffffu, cnt, 15), tl = __shfl_sync(0xffffffffu, cnt, 31);
          const int ea = __shfl_sync(0xffffffffu, cnt, max(warp - 1, 0)), el = __shfl_sync(0xffffffffu, cnt, 16 + max(warp - 1, 0));
          const int pa = base_all + (warp > 0 ? ea : 0), pl_ = base_loc + (warp > 0 ? el : 0);
          if (t) {
            const unsigned lt = (1u << lane) - 1u;
            const int ga = pa + __popc(bal & lt);
            gci()[r] = (short)ga;
            if (r % nc == crank) {
              const int ll = pl_ + __popc(bal & mine_mask & lt);
              lci()[r / nc] = (short)ll;
              tloc()[ll] = (unsigned short)r;
            }
          }
          base_all += ta;
          base_loc += tl;
          wsync();
        }
        n_touched = base_all;
        n_touched_local = base_loc;
      }
      // ---- 4. scatter: delta of the touched rows on the tensor cores, 128 compacted rows per pass
      const int n_pass = ceil_div(n_touched_local, 128);
      if (tid == 0) bars->n_pass = n_pass;
      if (n_pass == 0) {
        signal_issuer();
        ++n_sc;  // the issuer still commits once
        // No row of this CTA was touched: every MMA that read the block buffers has been read back, only the clearing
        // copy may still be on its way.
        if (tid == kLoaderThread && u + 1 < a.n_plan) {
          const bool okl = fast ? wait(&bars->zero_done, n_zero & 1, a.wait_limit, abort) : true;
          if (okl) issue_block_loads(smem, lay, bars, map_pk, map_gk, row, a.n_tok, C, u + 1);  // (a wait that ran out shows up at the next one)
        }
      }
      bool okz = true;
      for (int p = 0; p < n_pass; ++p) {
        {  // one-hot operand [C/64][128 rows][64 tokens] (in the buffer of the prepared keys, which are dead by now)
          if (p > 0) {  // a further pass: clear what the previous one set
            uint4* o = reinterpret_cast<uint4*>(smem + lay.P);
            for (int i = tid; i < C * 16; i += kWorkers) o[i] = make_uint4(0, 0, 0, 0);
            wsync();
          }
          if (p == 0 && fast) okz = wait(&bars->zero_done, n_zero & 1, a.wait_limit, abort);  // the cleared buffer has landed
          if (okz && my >= 0 && my % nc == crank) {
            const int ll = lci()[my / nc] - p * 128;
            if (ll >= 0 && ll < 128) {
              const uint32_t off = (uint32_t)(tid >> 6) * (128u * 128u) + tc::sw128_offset(ll, tid & 63);
              *reinterpret_cast<unsigned short*>(smem + lay.P + off) = 0x3F80;  // bf16 1.0
            }
          }
        }
        signal_issuer();
        // this thread's share of the epilogue: row = accumulator lane quarter*32 + lane, 32 of its 128 elements
        const int quarter = warp & 3, colq = warp >> 2;
        const int ci = quarter * 32 + lane;
        const bool act = p * 128 + ci < n_touched_local;
        const int r = act ? tloc()[p * 128 + ci] : 0;
        const size_t grow = (size_t)row * a.capacity + r;
        uint4 old[4];
        if (act) {
#pragma unroll
          for (int j = 0; j < 4; ++j) old[j] = *reinterpret_cast<const uint4*>(a.k_sum + grow * HD + colq * 32 + j * 8);
        }
        ok = wait(&bars->sc_done, n_sc & 1, a.wait_limit, abort) && okz;
        ++n_sc;
        // The scatter was the last reader of the block buffers: one thread has the next block copied in right away (both
        // operands of every block, also where an update needs only one: the two barriers stay in step).
        if (ok && p == n_pass - 1 && tid == kLoaderThread && u + 1 < a.n_plan)
          issue_block_loads(smem, lay, bars, map_pk, map_gk, row, a.n_tok, C, u + 1);
        if (!wvote(ok)) return false;
        tc::tc_fence_after_sync();
        float x[32];
        {
          uint32_t d[32];
          tc::tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(colq * 32), d);
          tc::tmem_ld_wait();
          tc::tc_fence_before_sync();
          // row = bf16(row + bf16(delta)) on packed pairs: one conversion per two elements (conversions are the
          // slowest instructions of this loop), the sum of two bf16 numbers rounded once
          float s1 = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t w4[4] = {old[j].x, old[j].y, old[j].z, old[j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int c = j * 8 + e * 2;
              const __nv_bfloat162 dl = __floats2bfloat162_rn(__uint_as_float(d[c]), __uint_as_float(d[c + 1]));
              uint32_t ow = act ? w4[e] : 0u;
              const __nv_bfloat162 sum = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&ow), dl);
              const float2 f2 = __bfloat1622float2(sum);
              x[c] = f2.x;
              x[c + 1] = f2.y;
              s1 += f2.x + f2.y;
            }
          }
          stat(0)[colq * 128 + ci] = s1;
        }
        if (act) {  // the carried sums
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16(x[j * 8 + 0], x[j * 8 + 1]); o.y = pack_bf16(x[j * 8 + 2], x[j * 8 + 3]);
            o.z = pack_bf16(x[j * 8 + 4], x[j * 8 + 5]); o.w = pack_bf16(x[j * 8 + 6], x[j * 8 + 7]);
            *reinterpret_cast<uint4*>(a.k_sum + grow * HD + colq * 32 + j * 8) = o;
          }
        }
        wsync();
        const float mean = (stat(0)[ci] + stat(0)[128 + ci] + stat(0)[256 + ci] + stat(0)[384 + ci]) * (1.0f / HD);
        float s2 = 0.f;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          x[c] -= mean;
          s2 += x[c] * x[c];
        }
        stat(1)[colq * 128 + ci] = s2;
        wsync();
        const float var = (stat(1)[ci] + stat(1)[128 + ci] + stat(1)[256 + ci] + stat(1)[384 + ci]) * (1.0f / HD);
        const float rstd = 1.0f / sqrtf(var + a.L.ln_eps);
        if (act) {
          const int l = r / nc;
          const int slot = pool_next + gci()[r];
          bf16* pdst = a.pool_k ? a.pool_k + ((size_t)row * a.pool_rows + slot) * HD + colq * 32 : nullptr;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float y[8];
            const float4 w0 = *reinterpret_cast<const float4*>(ln_w + colq * 32 + j * 8), w1 = *reinterpret_cast<const float4*>(ln_w + colq * 32 + j * 8 + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(ln_b + colq * 32 + j * 8), b1 = *reinterpret_cast<const float4*>(ln_b + colq * 32 + j * 8 + 4);
            const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w}, bv8[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = x[j * 8 + e] * rstd * wv[e] + bv8[e];
            uint4 o;
            o.x = pack_bf16(y[0], y[1]); o.y = pack_bf16(y[2], y[3]); o.z = pack_bf16(y[4], y[5]); o.w = pack_bf16(y[6], y[7]);
            *reinterpret_cast<uint4*>(smem + lay.R + piece(lay.Rcap, l, colq * 4 + j)) = o;
            if (pdst) *reinterpret_cast<uint4*>(pdst + j * 8) = o;
          }
        }
      }
      if (fast) ++n_zero;
      // ---- 5. the version: every touched row moved to a fresh pool row
      for (int i = tid; i < S1; i += kWorkers)
        if (tf()[i] == (unsigned short)u) cur()[i] = pool_next + gci()[i];
      pool_next += n_touched;
      wsync();
      if (ver)
        for (int i = tid + crank * kWorkers; i < S1; i += kWorkers * nc) ver[i] = cur()[i];
      ++n_load;
      signal_issuer();  // the resident memory is final for the next update
    }
    // final attention view of the keys, row order, for whoever continues from this memory (the decode cache)
    {
      const kvm_update_plan pl = a.plan[a.n_plan - 1];
      const int S = pl.state_before + pl.n_append;
      for (int i = tid; i < n_local(S, nc, crank) * 16; i += kWorkers) {
        const int l = i >> 4, c = i & 15;
        const int r = l * nc + crank;
        *reinterpret_cast<uint4*>(a.k_attn + ((size_t)row * a.capacity + r) * HD + c * 8) =
            *reinterpret_cast<const uint4*>(smem + lay.R + piece(lay.Rcap, l, c));
      }
    }
    return true;
  }
};

struct Maps {
  CUtensorMap pk, gk;  // [rows * n_tok][D] bf16, boxes of 64 elements x C tokens
};

__global__ void __launch_bounds__(kThreads, 1)
kvm_chain_tc_kernel(const __grid_constant__ Args a, const __grid_constant__ Maps maps, const __grid_constant__ vside::DeltaArgs va,
                    const __grid_constant__ vside::Maps vmaps) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(16) float ln_s[2 * HD];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((int)blockIdx.x >= a.chain_ctas) {
    // A spare CTA of the launch (whole clusters of them): it works on the value side of the updates the routing has
    // published so far, until the routing is over; what is left then is taken by the kernel behind this one.
    if (tid < vside::kThreads) vside::delta_jobs(va, vmaps, smem, tid);
    return;
  }
  const int nc = a.nc;
  const int row = blockIdx.x / nc, crank = blockIdx.x % nc;
  const Layout lay(a.L.C, a.s_max, nc);
  Bars* bars = reinterpret_cast<Bars*>(smem + lay.bars);
  const bool aligned = (tc::smem_u32(smem) & 1023u) == 0;  // operand tiles need 1024-byte alignment (uniform over the grid)
  if (!aligned) {
    if (tid == 0) {
      atomicExch(a.status, KVM_ERR_UNSUPPORTED);
      if (a.chain_done) atomicAdd(a.chain_done, 1);
    }
    return;
  }
  for (int i = tid; i < HD; i += kThreads) {
    ln_s[i] = a.L.ln_w[i];
    ln_s[HD + i] = a.L.ln_b[i];
  }
  {  // resident memory starts as zeros: rows past the live ones feed the MMAs, too (their scores are masked)
    uint4* r4 = reinterpret_cast<uint4*>(smem + lay.R);
    for (int i = tid; i < lay.Rcap * 16; i += kThreads) r4[i] = make_uint4(0, 0, 0, 0);
    for (int i = tid; i < a.s_max; i += kThreads) reinterpret_cast<int*>(smem + lay.rowi)[i] = 0;
    unsigned short* stamps = reinterpret_cast<unsigned short*>(smem + lay.tloc + ((2u * a.L.C + 15u) & ~15u));
    for (int i = tid; i < a.s_max; i += kThreads) stamps[i] = 0;  // update numbers start at 1
  }
  if (tid == 0) {
    tc::mbar_init(&bars->full_p, 1);
    tc::mbar_init(&bars->full_g, 1);
    for (int i = 0; i < 2; ++i) {
      for (int hb = 0; hb < 2; ++hb) {
        tc::mbar_init(&bars->tm_full[hb][i], 1);
        tc::mbar_init(&bars->tm_empty[hb][i], 8);  // the eight warps that read a token tile
      }
    }
    tc::mbar_init(&bars->w2i, kWorkerWarps);
    tc::mbar_init(&bars->sc_done, 1);
    tc::mbar_init(&bars->xbar[0], 1);  // one local arrival that states the bytes the peers will store
    tc::mbar_init(&bars->xbar[1], 1);
    tc::mbar_init(&bars->zero_done, 1);
    bars->abort = 0;
    bars->n_pass = 0;
    tc::fence_barrier_init();
  }
  if (warp == kWorkerWarps) tc::tmem_alloc(&bars->tmem_base, kTmemCols);
  tc::fence_proxy_async();
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  if (nc > 1) cluster_barrier();  // the peers' barriers exist before anybody arrives on them
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort = &bars->abort;

  bool ok = true;
  if (warp >= kWorkerWarps) {
    if (lane == 0) {
      Issuer is{a, smem, lay, bars, tmem, crank, row, &maps.pk, &maps.gk, warp - kWorkerWarps};
      is.abort = abort;
      ok = is.run();
    }
  } else {
    Workers w{a, smem, lay, bars, tmem, crank, row, ln_s, ln_s + HD, abort, tid, warp, lane, &maps.pk, &maps.gk};
    ok = w.run();
  }
  if (!ok) {
    // report, tell everybody in the cluster, then leave through the common exit
    atomicExch(a.status, KVM_ERR_DEVICE_TIMEOUT);
    *abort = 1;
    if (nc > 1 && lane == 0)
      for (int p = 0; p < nc; ++p)
        if (p != crank) st_peer_b32(peer_addr(&bars->abort, p), 1);
  }
  __syncwarp();
  __syncthreads();
  if (*abort) {
    // copies and MMAs of this CTA may still be in flight: they complete on their own within microseconds
    for (int k2 = 0; k2 < 64; ++k2) __nanosleep(1000);
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == kWorkerWarps) tc::tmem_dealloc(tmem, kTmemCols);
  if (tid == 0 && a.chain_done) {  // (the spare CTAs stop taking value-delta jobs when every routing CTA has got here)
    __threadfence();
    atomicAdd(a.chain_done, 1);
  }
  if (nc > 1) cluster_barrier();  // nobody leaves while a peer may still write into its shared memory
}

// ------------------------------------------------------------------------------------------------ value side
constexpr int kVpWarps = 16;
constexpr int kVpQueue = 4;  // routed tokens of a row whose value rows are fetched together

// One warp per memory row.  route: [rows][n_plan][C] (>= 0: merged into that row, -(1+r): appended as row r).
// The warp walks the decisions of all updates (a tile of them at a time in shared memory), queues the tokens that
// concern its row and fetches their value rows kVpQueue at a time (the loads are independent, the sums are formed
// afterwards in token order), so that the walk is bound by throughput and not by the latency of one row.
__global__ void __launch_bounds__(kVpWarps * 32, 2)
kvm_vpass_kernel(LayerDev L, Tensor4 v, Tensor4 gate, const kvm_update_plan* __restrict__ plan, int n_plan,
                 const int* __restrict__ route, MemoryDev mem, bf16* __restrict__ pool_v, long long pool_rows,
                 const int* __restrict__ ver_idx, long long ver_rows, int s_final, int tile_updates,
                 const int* __restrict__ status) {
  if (*status != 0) return;  // the chain gave up: its routing decisions and version tables are not to be trusted
  extern __shared__ __align__(16) unsigned char vsm[];
  short* rt = reinterpret_cast<short*>(vsm);                                        // [tile_updates][C] decisions of the tile
  int* vrow = reinterpret_cast<int*>(vsm + (size_t)tile_updates * L.C * 2);         // [n_plan] version_row of every update
  const int C = L.C, EPL = C / 32;            // EPL tokens per lane: 4 or 8
  const int log2c = C == 256 ? 8 : 7;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = blockIdx.y;
  const int b = row / L.Hkv, h = row % L.Hkv;
  const int r = blockIdx.x * kVpWarps + warp;  // this warp's memory row
  const bool live = r < s_final;
  const bool versions = pool_v != nullptr && ver_idx != nullptr;
  const int* route_row = route + (size_t)row * n_plan * C;
  const int* ver_row = ver_idx + (size_t)row * ver_rows + r;
  const bf16* v_base = v.row(b, h, 0) + lane * 4;
  const bf16* g_base = gate.row(b, h, 0);
  bf16* pool_row = pool_v + (size_t)row * pool_rows * HD + lane * 4;
  const bool gate_values = L.gate_values != 0;
  float x[4] = {0.f, 0.f, 0.f, 0.f};           // carried value sum of the row (bf16 values), elements 4*lane..
  float acc[4] = {0.f, 0.f, 0.f, 0.f};         // sum of the gated values of the update being collected
  float vl = 0.f;
  int acc_u = -1, acc_slot = -1, nq = 0;
  int q0 = 0, q1 = 0, q2 = 0, q3 = 0;          // queued tokens (bit 30: appended); the same in every lane
  bool born = false;
  for (int i = tid; i < n_plan; i += kVpWarps * 32) vrow[i] = plan[i].version_row;

  // the value view of the row after the update being collected: normalize(sum) * magnitude, into the pool row of that version
  auto finalize = [&]() {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[i] = bf16_round(x[i] + bf16_round(acc[i]));
      acc[i] = 0.f;
    }
    if (acc_slot >= 0) {
      const float n2 = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
      const float nrm = fmaxf(sqrtf(warp_sum(n2)), 1e-12f);
      float y[4] = {x[0], x[1], x[2], x[3]};
      divide_by(y, nrm);
      uint2 o;
      o.x = pack_bf16(y[0] * vl, y[1] * vl);
      o.y = pack_bf16(y[2] * vl, y[3] * vl);
      *reinterpret_cast<uint2*>(pool_row + (size_t)acc_slot * HD) = o;
    }
    acc_u = -1;
  };
  // fetch the queued tokens' value rows (and gates, and the pool slots of their updates) together, then apply in order
  auto flush = [&]() {
    const int item[kVpQueue] = {q0, q1, q2, q3};
    uint2 raw[kVpQueue];
    bf16 g[kVpQueue];
    int slot[kVpQueue];
#pragma unroll
    for (int i = 0; i < kVpQueue; ++i) {
      if (i < nq) {
        const int t = item[i] & 0x3fffffff;
        raw[i] = *reinterpret_cast<const uint2*>(v_base + (long long)t * v.st);
        g[i] = g_base[(long long)t * gate.st];
        const int vr = vrow[t >> log2c];
        slot[i] = (versions && vr >= 0) ? ver_row[vr] : -1;
      }
    }
#pragma unroll
    for (int i = 0; i < kVpQueue; ++i) {
      if (i < nq) {
        const int u = (item[i] & 0x3fffffff) >> log2c;
        if (acc_u >= 0 && acc_u != u) finalize();
        const float2 p0 = unpack_bf16(raw[i].x), p1 = unpack_bf16(raw[i].y);
        float o[4] = {p0.x, p0.y, p1.x, p1.y};
        const float gf = __bfloat162float(g[i]);
        if (item[i] & 0x40000000) {
          // the row is born from this token: value (gated where the layer says so) and magnitude
          const bool gated = u == 0 ? (L.gate_initial != 0) : (L.gate_appends != 0 && gate_values);
          if (u > 0 && gated) {
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = bf16_round(o[e] * gf);
          }
          vl = sqrtf(warp_sum(o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3]));  // initial rows: of the ungated value
#pragma unroll
          for (int e = 0; e < 4; ++e) x[e] = (u == 0 && gated) ? bf16_round(o[e] * gf) : o[e];
          born = true;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[e] += gate_values ? bf16_round(o[e] * gf) : o[e];
        }
        acc_u = u;
        acc_slot = slot[i];
      }
    }
    nq = 0;
  };
  auto push = [&](int item) {
    if (nq == 0) q0 = item;
    else if (nq == 1) q1 = item;
    else if (nq == 2) q2 = item;
    else q3 = item;
    if (++nq == kVpQueue) flush();
  };

  for (int u0 = 0; u0 < n_plan; u0 += tile_updates) {
    const int nu = min(tile_updates, n_plan - u0);
    __syncthreads();
    for (int i = tid; i < nu * C; i += kVpWarps * 32) rt[i] = (short)route_row[(size_t)u0 * C + i];
    __syncthreads();
    if (!live) continue;
    const unsigned want_m = (unsigned)(r & 0xffff) * 0x10001u, want_a = (unsigned)((-(1 + r)) & 0xffff) * 0x10001u;
    for (int uu = 0; uu < nu; ++uu) {
      const int u = u0 + uu;
      // two decisions per 32-bit word; token 2j of this lane's share in the low half of word j
      const unsigned* w = reinterpret_cast<const unsigned*>(rt + uu * C + lane * EPL);
      unsigned e4[4];
      if (EPL == 8) {
        const uint4 q4 = *reinterpret_cast<const uint4*>(w);
        e4[0] = q4.x; e4[1] = q4.y; e4[2] = q4.z; e4[3] = q4.w;
      } else {
        const uint2 q2w = *reinterpret_cast<const uint2*>(w);
        e4[0] = q2w.x; e4[1] = q2w.y;
        e4[2] = e4[3] = 0x80008000u;  // matches no row
      }
      // bit j: token 2j, bit 16 + j: token 2j + 1
      unsigned m_app = 0, m_mrg = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        m_app |= (__vcmpeq2(e4[j], want_a) & 0x00010001u) << j;
        m_mrg |= (__vcmpeq2(e4[j], want_m) & 0x00010001u) << j;
      }
      if (u == 0) m_mrg = 0;
      unsigned any = __ballot_sync(0xffffffffu, (m_app | m_mrg) != 0);
      while (any) {  // lanes in order = tokens in order
        const int src = __ffs(any) - 1;
        any &= any - 1;
        const unsigned ma = __shfl_sync(0xffffffffu, m_app, src);
        unsigned mm = __shfl_sync(0xffffffffu, m_mrg, src) | ma;
        const int t0 = (u << log2c) + src * EPL;
        while (mm) {  // next token of the lane: the lower of (2 * first low bit, 2 * first high bit + 1)
          const unsigned lo = mm & 0xffffu, hi = mm >> 16;
          const int jl = lo ? 2 * (__ffs(lo) - 1) : 64, jh = hi ? 2 * (__ffs(hi) - 1) + 1 : 64;
          const int j = min(jl, jh);
          const unsigned bit = 1u << ((j >> 1) + ((j & 1) << 4));
          mm &= ~bit;
          push((t0 + j) | ((ma & bit) ? 0x40000000 : 0));
        }
      }
    }
  }
  if (live) {
    flush();
    if (acc_u >= 0) finalize();
  }
  if (live && born) {  // the carried state and its final view
    const size_t off = ((size_t)row * mem.capacity + r) * HD + lane * 4;
    uint2 s;
    s.x = pack_bf16(x[0], x[1]);
    s.y = pack_bf16(x[2], x[3]);
    *reinterpret_cast<uint2*>(mem.v_sum + off) = s;
    if (lane == 0) mem.vlen[(size_t)row * mem.capacity + r] = vl;
    const float n2 = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    const float nrm = fmaxf(sqrtf(warp_sum(n2)), 1e-12f);
    float y[4] = {x[0], x[1], x[2], x[3]};
    divide_by(y, nrm);
    uint2 o;
    o.x = pack_bf16(y[0] * vl, y[1] * vl);
    o.y = pack_bf16(y[2] * vl, y[3] * vl);
    *reinterpret_cast<uint2*>(mem.v_attn + off) = o;
  }
}

}  // namespace chain

// ------------------------------------------------------------------------------------------------ host side
// Cluster size for `rows` kv rows: the largest size (<= 8) that fits shared memory and whose clusters are all
// resident at once; if none is, the smallest that fits (the rows then run in waves).  0: the shape does not fit.
static int chain_tc_cluster_size(int C, int s_max, int rows) {
  using namespace chain;
  static std::mutex mu;
  static int fit[64][4][2];      // [device][log2 nc][C == 256]: co-resident clusters, 0 = not asked yet
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int smallest = 0, best = 0;
  for (int lg = 0; lg <= 3; ++lg) {
    const int nc = 1 << lg;
    const Layout lay(C, s_max, nc);
    if (lay.total > (uint32_t)kMaxSmem) continue;
    if (!smallest) smallest = nc;
    int n_clusters;
    {
      std::lock_guard<std::mutex> lock(mu);
      n_clusters = fit[dev][lg][C == 256];
    }
    if (n_clusters == 0) {
      // the answer depends on the shared-memory size only through "one CTA per SM": ask with the largest size
      cudaLaunchConfig_t cfg = {};
      cfg.blockDim = dim3(kThreads);
      cfg.gridDim = dim3(nc * 64);
      cfg.dynamicSmemBytes = 200 * 1024;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = nc;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      if (cudaFuncSetAttribute(kvm_chain_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem) != cudaSuccess ||
          cudaOccupancyMaxActiveClusters(&n_clusters, kvm_chain_tc_kernel, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        n_clusters = -1;
      }
      if (n_clusters == 0) n_clusters = -1;
      std::lock_guard<std::mutex> lock(mu);
      fit[dev][lg][C == 256] = n_clusters;
    }
    if (n_clusters >= rows) best = nc;
  }
  return best ? best : smallest;
}

bool chain_tc_supported(int D, const LayerDev& L, int n_plan, int s_max, int rows) {
  if (D != 128 || (L.C != 128 && L.C != 256) || n_plan < 2 || s_max >= 32000) return false;
  if (L.gate_initial && !L.gate_keys) return false;  // the pre-pass only writes gated keys for layers that gate keys
  return chain_tc_cluster_size(L.C, s_max, rows) > 0;
}

// The chain for one batch: routing + key side, then the value side.  pk_all / gk_all: [rows][n_plan*C][D] from the
// pre-pass; route: [rows][n_plan][C].
bool vside_setup(const LayerDev& L, int batch, long long T, Tensor4 v, Tensor4 gate, const kvm_update_plan* plan_dev, int n_plan,
                 int s_max, bf16* pool_v, long long pool_rows, const int* ver_idx, long long ver_rows, const int* route,
                 unsigned* tbits, int* status, uint32_t wait_limit, vside::DeltaArgs* a, vside::Maps* maps);
size_t vside_smem_bytes(int C, int s_max);
cudaError_t launch_vside(vside::DeltaArgs a, const vside::Maps& maps, Tensor4 v, MemoryDev mem, const int* born, cudaStream_t stream);

cudaError_t launch_chain_tc(const LayerDev& L, int batch, long long T, Tensor4 v, Tensor4 gate, const kvm_update_plan* plan_dev,
                            int n_plan, int s_max, MemoryDev mem, bf16* pool_k, bf16* pool_v, long long pool_rows, int* ver_idx,
                            long long ver_rows, const bf16* pk_all, const bf16* gk_all, int* route, int* born, unsigned* tbits,
                            int* status, uint32_t wait_limit, uint32_t test_flags, cudaStream_t stream) {
  using namespace chain;
  const int rows = batch * L.Hkv, C = L.C;
  const int nc = chain_tc_cluster_size(C, s_max, rows);
  if (nc <= 0) return cudaErrorInvalidConfiguration;
  const Layout lay(C, s_max, nc);
  const long long n_tok = (long long)n_plan * C;
  Maps maps;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)((long long)rows * n_tok)};
    const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)C};
    if (!encode_bf16_map(&maps.pk, pk_all, 2, dims, strides, box) || !encode_bf16_map(&maps.gk, gk_all, 2, dims, strides, box))
      return cudaErrorInvalidValue;
  }
  Args a;
  a.L = L; a.plan = plan_dev; a.n_plan = n_plan; a.nc = nc; a.s_max = s_max; a.n_tok = n_tok;
  a.k_sum = mem.k_sum; a.k_attn = mem.k_attn; a.capacity = mem.capacity;
  a.pool_k = ver_idx ? pool_k : nullptr; a.pool_rows = pool_rows; a.ver_idx = ver_idx; a.ver_rows = ver_rows;
  a.route = route; a.born = born; a.status = status; a.wait_limit = wait_limit; a.test_flags = test_flags;
  a.progress = nullptr; a.chain_done = nullptr; a.chain_ctas = rows * nc;
  // The value side (with versions): deltas of every (kv row, update) on the tensor cores, then one warp per memory row.
  // SMs the routing leaves free take value-delta jobs inside the same launch, as whole clusters behind the routing's,
  // following the routing through a flag per (kv row, CTA); three control words and the flags live behind the bit table.
  const bool vside_on = ver_idx && pool_v;
  vside::DeltaArgs va = {};
  vside::Maps vmaps = {};
  int spare = 0;
  size_t smem_bytes = lay.total;
  cudaError_t e;
  if (vside_on) {
    if (!vside_setup(L, batch, T, v, gate, plan_dev, n_plan, s_max, pool_v, pool_rows, ver_idx, ver_rows, route, tbits, status,
                     wait_limit, &va, &vmaps))
      return cudaErrorInvalidValue;
    // control words: job counter, finished routing CTAs, given-back jobs (count, taken), then the progress flags and
    // the list of given-back jobs (one per spare CTA at most)
    int* ctrl = reinterpret_cast<int*>(tbits + (size_t)rows * n_plan * va.words);
    e = cudaMemsetAsync(ctrl, 0, (size_t)(4 + rows * nc) * sizeof(int), stream);
    if (e != cudaSuccess) return e;
    va.queue = ctrl;
    int dev = 0, n_sm = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    spare = std::max(0, (n_sm - rows * nc) / nc) * nc;
    if (vside_smem_bytes(C, s_max) > (size_t)kMaxSmem) spare = 0;
    if (spare > 0) {
      a.chain_done = ctrl + 1;
      a.progress = ctrl + 4;
      va.n_given_back = ctrl + 2;
      va.given_back_taken = ctrl + 3;
      va.given_back = ctrl + 4 + rows * nc;
      va.chain_done = a.chain_done;
      va.progress = a.progress;
      va.nc = nc;
      va.chain_ctas = rows * nc;
      smem_bytes = std::max(smem_bytes, vside_smem_bytes(C, s_max));
    }
  }
  e = cudaFuncSetAttribute(kvm_chain_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads);
  cfg.gridDim = dim3(rows * nc + spare);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nc;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kvm_chain_tc_kernel, a, maps, va, vmaps);
  if (e != cudaSuccess) return e;
  if (vside_on) return launch_vside(va, vmaps, v, mem, born, stream);
  // Without (only the final memory is wanted): one warp per memory row walks the routing decisions itself, as many
  // updates as fit 64 KB per tile
  const int tile_updates = std::max(1, std::min(n_plan, (64 * 1024) / (C * 2)));
  const size_t vsmem = (size_t)tile_updates * C * 2 + (size_t)((n_plan + 3) & ~3) * 4;
  e = cudaFuncSetAttribute(kvm_vpass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)vsmem);
  if (e != cudaSuccess) return e;
  dim3 vgrid((unsigned)ceil_div(s_max, kVpWarps), rows);
  kvm_vpass_kernel<<<vgrid, kVpWarps * 32, vsmem, stream>>>(L, v, gate, plan_dev, n_plan, route, mem, ver_idx ? pool_v : nullptr,
                                                            pool_rows, ver_idx, ver_rows, s_max, tile_updates, status);
  return cudaGetLastError();
}

}  // namespace kvm
