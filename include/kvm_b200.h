/*
 * kvm_b200 -- C ABI of the B200 (sm_100a) Key-Value-Means sequence-mixer kernels.
 *
 * The reference project (SmerkyG/KVM-paper) has no FFI: its mixer is a Python class and its device
 * code is Triton-in-Python.  The entry points below are what a binding for that hot path binds
 * instead; each one cites the reference interface it replaces (path inside the reference project).
 *
 * Conventions
 *   - every pointer named *_dev / documented "device" is a CUDA device pointer owned by the caller;
 *     the library allocates no device memory.  What it keeps between calls, per process: the text of the
 *     calling thread's last error; per device, created on first use and guarded by mutexes so that several
 *     host threads may drive several GPUs: one side stream with two events (kvm_decode_step's overlapped
 *     memory update), a small cache of tensor maps keyed by the decode cache's addresses and sizes, the
 *     shared-memory limits already raised on the kernels, cached occupancy answers, and the device address
 *     of the built-in scratch of kvm_decode_step_static.  None of it depends on the data of a call;
 *   - all activations and memory rows are bfloat16, lengths/norms fp32, indices int32;
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream); calls only enqueue work;
 *   - return value 0 = ok, otherwise one of KVM_ERR_*; kvm_last_error_string() describes the last
 *     failure of the calling thread.  Argument errors are detected before anything is launched.
 *   - "kv row" = one (batch, kv-head) pair, index b*Hkv + h;  "q row" = b*Hq + h.
 */
#ifndef KVM_B200_H_
#define KVM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVM_OK 0
#define KVM_ERR_BAD_ARGUMENT 1
#define KVM_ERR_CAPACITY 2
#define KVM_ERR_DEVICE_TIMEOUT 3
#define KVM_ERR_CUDA 4
#define KVM_ERR_UNSUPPORTED 5

/* Static description of one mixer layer: the fields the reference mixer reads from its config and
 * parameters (model/kvm_mixer.py:79-118).  Device arrays are read by the kernels. */
typedef struct kvm_layer {
  int32_t n_q_heads;      /* Hq */
  int32_t n_kv_heads;     /* Hkv, divides Hq */
  int32_t head_dim;       /* D == Dv, one of 32, 64, 128 */
  int32_t chunk_len;      /* C, block length; multiple of 16, <= 512 */
  int32_t n_bswa_chunks;  /* W, blocks in the sliding window (>= 1) */
  int32_t rope_dim;       /* leading key dims zeroed before the memory LayerNorm */
  int32_t sink_len;       /* protected leading memory rows */
  int32_t gate_keys;      /* kvm_use_merge_gate_keys */
  int32_t gate_values;    /* kvm_use_merge_gate_values */
  int32_t gate_appends;   /* kvm_apply_merge_gate_to_appends */
  int32_t gate_initial;   /* kvm_apply_merge_gate_to_initial_state */
  float ln_eps;           /* eps of ln_s_k */
  const float* ln_weight_dev;   /* [D] fp32 copy of ln_s_k.weight */
  const float* ln_bias_dev;     /* [D] */
  const float* front_temp_dev;  /* [Hq] front_head_temp (ones if head temps are off) */
  const float* state_temp_dev;  /* [Hq] state_head_temp */
} kvm_layer;

/* A strided bf16 tensor [B, H, T, D] with the last dimension contiguous (strides in elements).
 * The reference hands the mixer transposed views of [B,T,H,D] projections (model/kvm_mixer.py:397-399). */
typedef struct kvm_tensor4 {
  const void* ptr;
  int64_t stride_b, stride_h, stride_t;
} kvm_tensor4;

/* The compressed memory of one layer for `n_rows` kv rows, `capacity` rows each (device). */
typedef struct kvm_memory {
  void* k_sum;    /* [n_rows, capacity, D] bf16  sums of prepared keys  (reference cache entry kvm_s_k) */
  void* v_sum;    /* [n_rows, capacity, D] bf16  sums of values         (kvm_s_v) */
  float* vlen;    /* [n_rows, capacity]    fp32  value magnitudes       (kvm_s_vlen) */
  void* k_attn;   /* [n_rows, capacity, D] bf16  LayerNorm(k_sum): the keys attention reads */
  void* v_attn;   /* [n_rows, capacity, D] bf16  normalize(v_sum)*vlen: the values attention reads */
  int32_t capacity;
} kvm_memory;

/* Per-update schedule entry (host computes it with the reference's own integer/float rules,
 * model/kvm_mixer.py:131-172; the kernels only see the table).  Update u consumes the token block
 * [u*C, (u+1)*C) and produces memory version u; version 0 is the initial memory. */
typedef struct kvm_update_plan {
  int32_t state_before;  /* rows before the update */
  int32_t n_append;      /* 0..C rows appended (the least similar tokens), the rest are merged */
  int32_t version_row;   /* first entry of the version written after this update inside the version tables
                            (one table entry per memory row: its row in the workspace's row pool) */
  int32_t reserved;
} kvm_update_plan;

/* Bytes of scratch kvm_prefill_forward needs for the given shape (row pool, version tables, prepared keys,
 * routing scratch, status word).
 * Replaces the workspace allocation inside build_prefill_forward
 * (model/kernels/kvm_triton_training_kernels.py:3416-3448). */
size_t kvm_prefill_workspace_bytes(const kvm_layer* layer, int32_t batch, int64_t seq_len,
                                   int64_t total_version_rows);

/* Whole-prompt prefill: front attention, block-recurrent memory updates and joint attention of
 * every query block over [memory version ; sliding window].
 * Replaces SequenceMixer.forward_prefill between the post-QKV tensors and the input of c_proj
 * (model/kvm_mixer.py:403-492, model/kvm_triton_mixer.py:560-611) and the Triton host driver
 * build_prefill_forward (model/kernels/kvm_triton_training_kernels.py:3386-3602).
 *   q [B,Hq,T,D], k,v [B,Hkv,T,D], gate [B,Hkv,T,1] (stride_t in elements, last dim 1)
 *   plan_dev     [n_updates+1] kvm_update_plan on the device; entry 0 describes the initial memory
 *                (state_before = 0, n_append = min(T,C), version_row = 0)
 *   plan_host    the same table in host memory (used for launch geometry only)
 *   memory       receives the final memory (capacity >= final length), n_rows = B*Hkv
 *   out          [B,T,Hq*D] bf16, contiguous
 *   route_dev    optional [B*Hkv, n_updates+1, C] int32: for every token of every consumed block the
 *                memory row it was merged into (>= 0) or -(1+row) if it was appended as that row
 *   phases       KVM_PREFILL_CHAIN | KVM_PREFILL_ATTENTION for the whole operator; one bit alone runs
 *                that phase only (attention alone needs the versions a chain run left in `workspace`)
 */
#define KVM_PREFILL_CHAIN 1u      /* run the memory chain (fills `memory`, the versions and route_dev) */
#define KVM_PREFILL_ATTENTION 2u  /* run block attention (reads the versions in `workspace`, fills out) */
#define KVM_PREFILL_LEGACY_ATTENTION 4u /* with ATTENTION: use the warp-level mma.sync kernel even where the
                                           tcgen05 kernel applies (head_dim 128, block multiple of 128) */
#define KVM_PREFILL_LEGACY_CHAIN 8u     /* with CHAIN: use the general chain kernel even where the kernel with the
                                           resident memory on the tensor cores applies (head_dim 128, block 128/256) */
#define KVM_PREFILL_TEST_WITHHOLD_ARRIVAL 16u /* test hook, with CHAIN on the tensor-core chain: one barrier arrival of
                                           the first update is withheld and the wait limit is a fraction of a
                                           millisecond, so that the bounded wait behind it runs out: the kernel must
                                           report KVM_ERR_DEVICE_TIMEOUT through kvm_prefill_status and return
                                           (nothing is in flight, nothing faults); the results are undefined */
int kvm_prefill_forward(const kvm_layer* layer, int32_t batch, int64_t seq_len,
                        kvm_tensor4 q, kvm_tensor4 k, kvm_tensor4 v, kvm_tensor4 gate,
                        const kvm_update_plan* plan_dev, const kvm_update_plan* plan_host,
                        int32_t n_updates, int64_t total_version_rows,
                        kvm_memory memory, void* out, int32_t* route_dev,
                        void* workspace, size_t workspace_bytes, uint32_t phases, void* stream);

/* kvm_prefill_forward for one rank of a head-sharded prefill whose block attention gathers the outputs by itself:
 * `layer` describes this rank's heads, `out_bases[r]` is rank r's whole output [B, T, n_ranks * Hq * D] bf16 (addresses
 * this process can write: its own buffer and peer mappings of the others'), and the attention kernel stores every
 * tile of this rank's heads into columns [rank * Hq * D, (rank + 1) * Hq * D) of ALL of them (peer stores over NVLink,
 * issued by the copy engine while other tiles are computed), so no collective follows.  A rank's buffer is complete
 * once every rank's call has finished: the caller synchronises the ranks behind the call (and before the buffers are
 * written again).  Needs the tensor-core attention kernel (head_dim 128, blocks of a multiple of 128 tokens).
 * No counterpart in the reference (it is data-parallel only). */
int kvm_prefill_forward_gathered(const kvm_layer* layer, int32_t batch, int64_t seq_len,
                                 kvm_tensor4 q, kvm_tensor4 k, kvm_tensor4 v, kvm_tensor4 gate,
                                 const kvm_update_plan* plan_dev, const kvm_update_plan* plan_host,
                                 int32_t n_updates, int64_t total_version_rows, kvm_memory memory,
                                 int32_t n_ranks, int32_t rank, void* const* out_bases, int32_t* route_dev,
                                 void* workspace, size_t workspace_bytes, uint32_t phases, void* stream);

/* Waits for `stream` and returns what the kernels of the last prefill on this workspace reported (the
 * status word is opened by a call that includes KVM_PREFILL_CHAIN and collects what that call and later
 * attention-only calls report): KVM_OK, or KVM_ERR_DEVICE_TIMEOUT if a bounded device-side wait
 * (mbarrier / tensor-memory pipeline) expired -- the kernels then leave through their normal exit, nothing
 * hangs, the output is undefined.  A reported status is cleared.  No counterpart in the reference (its
 * Triton kernels have no device-side waits). */
int kvm_prefill_status(void* workspace, void* stream);

/* Where kvm_prefill_forward keeps its intermediate results inside `workspace` (byte offsets), for inspection
 * after a call: the row pool of the memory's attention view ([B*Hkv, pool_rows, D] bf16, keys and values),
 * the version tables ([B*Hkv, total_version_rows] int32: entry plan[u].version_row + r is the pool row that
 * holds memory row r after update u) and the prepared keys of all consumed tokens
 * ([B*Hkv, (n_updates+1)*C, D] bf16; present when n_updates > 0; the gated keys lie in a second array of
 * the same shape).  Counterpart of the reference's
 * capture_state_snapshots hook (model/kernels/kvm_triton_training_kernels.py:3518-3524), without copies. */
typedef struct kvm_prefill_layout {
  size_t status_offset;
  size_t pool_k_offset;
  size_t pool_v_offset;
  size_t version_table_offset;
  size_t prepared_keys_offset;
  size_t gated_keys_offset;    /* bf16(prepared key * gate), same shape (head_dim 128 with blocks of 128 / 256 only) */
  int64_t pool_rows;
  size_t total_bytes;
} kvm_prefill_layout;
int kvm_prefill_workspace_layout(const kvm_layer* layer, int32_t batch, int64_t seq_len,
                                 int64_t total_version_rows, kvm_prefill_layout* out);

/* The mixer's prologue in one pass over the projection outputs: token shift, per-head LayerNorm of q and k, rotary
 * embedding, merge gate, and the prepared / gated keys of the tokens the memory updates will consume.
 * Replaces the elementwise part of calc_qkv (model/value_residual_mixin.py:219-235: apply_token_shift of
 * model/tokenshift.py:11-37, ln_q, ln_k) and of forward's prefix (model/kvm_mixer.py:381-399:
 * apply_rotary_embeddings of model/rwkv7_backbone.py:76-88, merge gate 1 + elu(key_weighting(x)), head-major views);
 * the projections themselves (c_q, c_k, c_v, key_weighting: plain GEMMs) and the value residual stay with the caller.
 * All tensors bf16 and contiguous unless said; every operation rounds to bf16 where the reference's bf16 module does.
 *   q_lin [B,T,Hq*D], k_lin, v_lin [B,T,Hkv*D]   projection outputs (v after a pre-shift value residual)
 *   gate_lin [B,T,Hkv]                            key_weighting output, NULL: gate of ones
 *   shift_q [Hq*D], shift_k, shift_v [Hkv*D]      token-shift scales, all three NULL: no token shift
 *   prev_q [B,Hq*D], prev_k, prev_v [B,Hkv*D]     last token of the previous call (cached decode), NULL: the first
 *                                                 token is shifted against itself
 *   ln_q_w, ln_q_b, ln_k_w, ln_k_b [D] fp32       per-head LayerNorm of q and k, all four NULL: none
 *   cos, sin [B or 1, T, D]                       rotary tables as RotaryEmbedding returns them (the sign of the
 *                                                 odd sin entries folded in); rope_stride_b = T*D or 0; NULL: none */
typedef struct kvm_prologue {
  const void* q_lin;
  const void* k_lin;
  const void* v_lin;
  const void* gate_lin;
  const void* shift_q;
  const void* shift_k;
  const void* shift_v;
  const void* prev_q;
  const void* prev_k;
  const void* prev_v;
  const float* ln_q_w;
  const float* ln_q_b;
  const float* ln_k_w;
  const float* ln_k_b;
  float ln_qk_eps;
  const void* cos;
  const void* sin;
  int64_t rope_stride_b;
} kvm_prologue;
/*   q_out [B,T,Hq,D], k_out, v_out [B,T,Hkv,D]   the operator's inputs (pass them on as [B,H,T,D] views)
 *   gate_out [B,Hkv,T]                           merge gate
 *   workspace  a prefill workspace for this shape (kvm_prefill_workspace_bytes) or NULL.  When given and the
 *              prompt has memory updates, the prepared keys (and, for the tensor-core chain, the gated keys) of
 *              the consumed tokens are written where kvm_prefill_forward keeps them, and a following
 *              kvm_prefill_forward on the same workspace may be given KVM_PREFILL_KEYS_PREPARED to skip its own
 *              pass over the keys (same bits either way). */
#define KVM_PREFILL_KEYS_PREPARED 32u /* with CHAIN: the workspace already holds the prepared keys (kvm_prologue_forward) */
int kvm_prologue_forward(const kvm_layer* layer, int32_t batch, int64_t seq_len, const kvm_prologue* in,
                         void* q_out, void* k_out, void* v_out, void* gate_out, int64_t total_version_rows,
                         void* workspace, size_t workspace_bytes, void* stream);

/* The decode-time cache of one layer for `batch` sequences with ragged lengths (all device memory,
 * caller-owned).  Replaces TritonKVMDecodeCache (model/kvm_triton_decode.py:34-400); unlike the
 * reference's cache, lengths are per sequence. */
typedef struct kvm_decode_cache {
  kvm_memory memory;      /* n_rows = batch*Hkv */
  void* ring_k;           /* [batch*Hkv, W*C, D] bf16: token t lives at slot t mod (W*C) */
  void* ring_v;           /* [batch*Hkv, W*C, D] bf16 */
  void* ring_gate;        /* [batch*Hkv, W*C]    bf16 */
  int32_t* total_len;     /* [batch] tokens seen so far (advanced by kvm_decode_step) */
  int32_t* state_len;     /* [batch] memory rows in use */
} kvm_decode_cache;

/* Bytes of scratch kvm_decode_step needs.  The first (batch*Hkv + batch + 1) int32 of the workspace -- split
 * counters, two launch counters and the status word -- must be ZERO before the first step (cudaMemset once
 * after allocating); the kernels leave the counters at zero, so later steps need no clearing. */
size_t kvm_decode_workspace_bytes(const kvm_layer* layer, int32_t batch, int32_t max_rows_per_seq);

/* One decode token for every sequence of the batch: append to the ring, run the memory update for
 * the sequences that cross a block boundary at this step, then joint attention over
 * [memory ; window].  Replaces SequenceMixer.forward_single / _decode_one_token
 * (model/kvm_mixer.py:572-713, model/kvm_triton_mixer.py:717-757, 902-929) and the kernels
 * write_recent_ring / gather_overflow / kvm_decode_attention (model/kernels/kvm_triton_decode.py).
 *   q [B,Hq,1,D], k,v [B,Hkv,1,D], gate [B,Hkv,1,1] as kvm_tensor4 (stride_t unused)
 *   n_append_dev  [batch] int32: -1 = no memory update for this sequence at this step, otherwise
 *                 the number of rows the update appends (host schedule); may be NULL when
 *                 any_update == 0
 *   any_update    host count of sequences with n_append_dev[b] >= 0 (0: launch no update kernel; a
 *                 negative value or one above batch means "some, count unknown").  With a known
 *                 count the update (and the attention of the updated sequences behind it) runs on a
 *                 stream owned by the library, next to the attention of the other sequences, and is
 *                 joined back into `stream` at the end of the call; all work of the call is ordered
 *                 after prior work in `stream` and before later work in it
 *   max_rows      upper bound of (memory rows + window rows) over the batch (launch geometry)
 *   out           [B,1,Hq*D] bf16
 *   route_dev     optional [batch*Hkv, C] int32, written for updated sequences (see prefill)
 */
int kvm_decode_step(const kvm_layer* layer, int32_t batch, kvm_decode_cache cache,
                    kvm_tensor4 q, kvm_tensor4 k, kvm_tensor4 v, kvm_tensor4 gate,
                    const int32_t* n_append_dev, int32_t any_update, int32_t max_rows,
                    void* out, int32_t* route_dev, void* workspace, size_t workspace_bytes,
                    void* stream);

/* Waits for `stream` and returns what the decode kernels that used `workspace` have reported since the last
 * call: KVM_OK or KVM_ERR_DEVICE_TIMEOUT (a bounded wait of the attention kernel's copy pipeline expired; the
 * kernel drained and returned, that token's output is undefined).  `layer` and `batch` as given to
 * kvm_decode_step (they locate the word).  workspace == NULL reads the built-in scratch of
 * kvm_decode_step_static on the current device.  A reported status is cleared.  No counterpart in the
 * reference. */
int kvm_decode_status(const kvm_layer* layer, int32_t batch, void* workspace, void* stream);

/* `n_steps` consecutive decode steps whose inputs are already on the device (teacher-forced or synthetic
 * decoding, as in the reference's kernel benchmark, which pre-generates the per-token q/k/v/gate:
 * scripts/kvm_benchmark/common.py:341-512, 684-709).  Step i reads q/k/v/gate at
 * base + i*step_stride elements, n_append_dev + i*batch, and writes out + i*batch*Hq*D; any_update_host
 * and max_rows_host ([n_steps], host memory) carry the per-step launch flags of kvm_decode_step.
 * Equivalent to calling kvm_decode_step n_steps times; exists so that the host loop costs two kernel
 * launches per token and nothing else (any_update_host[i] is the count described above). */
int kvm_decode_run(const kvm_layer* layer, int32_t batch, kvm_decode_cache cache, int32_t n_steps,
                   kvm_tensor4 q, kvm_tensor4 k, kvm_tensor4 v, kvm_tensor4 gate,
                   int64_t q_step_stride, int64_t kv_step_stride, int64_t gate_step_stride,
                   const int32_t* n_append_dev, const int32_t* any_update_host, const int32_t* max_rows_host,
                   void* out, void* workspace, size_t workspace_bytes, void* stream);

/* Same decode step for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Some hosts of this library only receive tensors and a stream from their runtime and are
 * not allowed to call cudaMalloc themselves -- a plug-in inside an inference server whose memory pool is
 * closed to plug-ins, a callback running while its framework forbids allocation, a process whose device
 * memory was handed out in full at start-up.  For them the scratch that kvm_decode_step takes as
 * `workspace` lives in a fixed array inside the library image instead: KVM_STATIC_SCRATCH_BYTES per GPU
 * that loads the library, held until the process exits.  The caller still passes the cache, inputs and
 * output.  No cudaMalloc / cudaFree or other allocating routine is called.
 *   - Shapes whose scratch (kvm_decode_workspace_bytes) exceeds KVM_STATIC_SCRATCH_BYTES are rejected
 *     with KVM_ERR_CAPACITY and a message naming both sizes; use kvm_decode_step then.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the one array, which keeps the previous call's contents (the
 *     part that must start at zero is cleared on the stream by every call): two calls whose kernels can
 *     overlap on the GPU -- different streams, or different threads -- race.  Serialise them on one stream.
 */
#define KVM_STATIC_SCRATCH_BYTES (32u << 20)
int kvm_decode_step_static(const kvm_layer* layer, int32_t batch, kvm_decode_cache cache,
                           kvm_tensor4 q, kvm_tensor4 k, kvm_tensor4 v, kvm_tensor4 gate,
                           const int32_t* n_append_dev, int32_t any_update, int32_t max_rows,
                           void* out, int32_t* route_dev, void* stream);

/* Build k_attn / v_attn from k_sum / v_sum / vlen for rows [0, state_len[b]) of every sequence
 * (used when a cache is initialised from the reference's eager cache layout).
 * Replaces the normalised-copy refresh in TritonKVMDecodeCache.reset_
 * (model/kvm_triton_decode.py:264-317). */
int kvm_memory_refresh(const kvm_layer* layer, int32_t batch, kvm_memory memory,
                       const int32_t* state_len_dev, void* stream);

/* Head order after an all-gather of head-sharded mixer outputs: src [n_shards][n_tokens][shard_bytes] (what
 * an all-gather of the ranks' [B*T, h_loc*D] outputs leaves) -> dst [n_tokens][n_shards][shard_bytes], i.e.
 * [B, T, H*D] with the heads in rank order.  shard_bytes a multiple of 16, both buffers 16-byte aligned.
 * No counterpart in the reference (its mixers run on one device); replaces a strided tensor copy in the host code. */
int kvm_interleave_shards(void* dst, const void* src, int32_t n_shards, int64_t n_tokens, int64_t shard_bytes, void* stream);

/* Description of the last error of the calling thread ("" if none). */
const char* kvm_last_error_string(void);

/* Library/ABI version (major*100 + minor). */
int kvm_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KVM_B200_H_ */
