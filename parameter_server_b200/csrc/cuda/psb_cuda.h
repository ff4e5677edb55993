// C ABI of libpsb_cuda.so: every hand-written sm_100a kernel of the library is
// reached through one of these launchers. All pointers are device pointers
// unless stated otherwise; launchers enqueue on `stream` and never allocate or
// synchronise. Return value: 0 on success, otherwise minus the cudaError (a few
// launchers document a non-negative payload instead).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PSB_MAX_SHARDS 16
typedef unsigned long long psb_u64;  // 64-bit keys (same ABI as uint64_t)

// ---------------------------------------------------------------- sort / localise
size_t psb_sort_scratch_bytes(uint32_t n, int begin_bit, int end_bit);
int psb_sort_pairs(const void* in, int in_kind, psb_u64 seed, psb_u64* keys_a, uint32_t* vals_a,
                   int vals_given, psb_u64* keys_b, uint32_t* vals_b, uint32_t n, int begin_bit,
                   int end_bit, void* scratch, uint32_t* status, uint32_t* where_out, int pack_pos_bits,
                   cudaStream_t stream);
int psb_localize2(const psb_u64* keys_a, const psb_u64* keys_b, const uint32_t* pos_a, const uint32_t* pos_b,
                  const uint32_t* where, uint32_t* csc_row, uint32_t n, const uint32_t* row_ptr, uint32_t n_rows,
                  uint32_t fixed_z, const float* vals, const psb_u64* bounds, int S, psb_u64* ukeys,
                  uint32_t* seg_off, uint32_t* csr_col, float* csc_val, uint32_t* flagbits, uint32_t* wordbase,
                  uint32_t* n_unique, uint32_t* own_off, void* scratch, int pack_pos_bits, cudaStream_t stream);
int psb_owner_offsets(const psb_u64* ukeys, const uint32_t* n_unique, const psb_u64* bounds, int S,
                      uint32_t* own_off, cudaStream_t stream);
// Gated forms: every kernel of the call returns at once unless the device word *gate is non-zero.
int psb_sort_pairs_gated(const void* in, int in_kind, psb_u64 seed, psb_u64* keys_a, uint32_t* vals_a,
                         int vals_given, psb_u64* keys_b, uint32_t* vals_b, uint32_t n, int begin_bit,
                         int end_bit, void* scratch, uint32_t* status, uint32_t* where_out, int pack_pos_bits,
                         const uint32_t* gate, cudaStream_t stream);
int psb_localize2_gated(const psb_u64* keys_a, const psb_u64* keys_b, const uint32_t* pos_a, const uint32_t* pos_b,
                        const uint32_t* where, uint32_t* csc_row, uint32_t n, const uint32_t* row_ptr,
                        uint32_t n_rows, uint32_t fixed_z, const float* vals, const psb_u64* bounds, int S,
                        psb_u64* ukeys, uint32_t* seg_off, uint32_t* csr_col, float* csc_val, uint32_t* flagbits,
                        uint32_t* wordbase, uint32_t* n_unique, uint32_t* own_off, void* scratch,
                        int pack_pos_bits, const uint32_t* gate, cudaStream_t stream);
int psb_owner_offsets_n(const psb_u64* ukeys, const uint32_t* n_unique, const psb_u64* bounds, int S, uint32_t n,
                        uint32_t* seg_off, uint32_t* own_off, const uint32_t* skip_when_set, cudaStream_t stream);
// Bucket-based localisation (bucket_localize.cu): groups the nonzeros by key without a full sort.
size_t psb_bucket_localize_scratch_bytes(uint32_t max_n);
int psb_bucket_localize(const void* in, int in_kind, psb_u64 seed, uint32_t n, int low_zero_bits,
                        const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z, const float* vals,
                        const psb_u64* bounds, int S, psb_u64* cold_words, uint32_t* cold_pos, uint32_t* hot_pos,
                        psb_u64* ukeys, uint32_t* seg_off, uint32_t* csr_col, uint32_t* csc_row, float* csc_val,
                        uint32_t* flagbits, uint32_t* wordbase, uint32_t* n_unique, uint32_t* own_off,
                        void* scratch, uint32_t* status, uint32_t* gate_out, cudaStream_t stream);
size_t psb_localize_scratch_bytes(uint32_t n);
int psb_localize(const psb_u64* sorted_keys, uint32_t* sorted_pos, uint32_t n,
                 const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z, const float* vals,
                 const psb_u64* bounds, int S, psb_u64* ukeys, uint32_t* seg_off,
                 uint32_t* csr_col, float* csc_val, uint32_t* flagbits, uint32_t* wordbase,
                 uint32_t* n_unique, uint32_t* own_off, void* scratch, cudaStream_t stream);

// ---------------------------------------------------------------- server shard table
// Optimiser selection for the scalar-value table.
// PSB_ALGO_KEEP consumes a push round without touching the stored values (buffered KVVector: the
// application reads the round out of the inboxes and decides what to do with it)
enum { PSB_ALGO_FTRL = 0, PSB_ALGO_ADAGRAD = 1, PSB_ALGO_SGD = 2, PSB_ALGO_SUM = 3, PSB_ALGO_KEEP = 4 };
enum { PSB_LR_CONSTANT = 0, PSB_LR_DECAY = 1 };
enum { PSB_LOSS_LOGIT = 0, PSB_LOSS_SQUARE_HINGE = 1 };
enum { PSB_QUANT_NONE = 0, PSB_QUANT_INT8 = 1, PSB_QUANT_FP16 = 2 };

typedef struct {
  int algo;      // PSB_ALGO_*
  int lr_type;   // PSB_LR_*
  float alpha, beta;
  float l1, l2;  // elastic-net penalty
} PsbOptimizer;

// What a worker needs to pull from S shards and compute margins (kernel F2).
typedef struct {
  int S;
  int insert;                 // 1: insert absent keys on pull (KVMap first touch); 2: skip the gather (w_local given)
  void* table[PSB_MAX_SHARDS];            // Entry* of shard s (local or peer-mapped)
  psb_u64 mask[PSB_MAX_SHARDS];          // capacity-1 of shard s
  psb_u64 key_begin[PSB_MAX_SHARDS];     // first key of shard s's range
  psb_u64 slot_mult[PSB_MAX_SHARDS];     // 0: hashed slots; else order-preserving multiplier
  const uint32_t* applied[PSB_MAX_SHARDS];  // shard s's "applied" counter (may be peer-mapped)
  uint32_t need_applied;      // bounded delay: wait until applied[s] >= need_applied
  const psb_u64* ukeys;
  const uint32_t* n_unique;
  const uint32_t* own_off;
  float* w_local;             // out: weight per unique key
  int32_t* slot_local;        // in/out (nullable): slot of each key in its owner's table, -1 if absent
  const uint32_t* key_hit;    // nullable device flag: 1 = same key list as last time, reuse slot_local
  float* grad_zero;           // nullable: zeroed per unique key (prepares the push)
  // margins (skipped when n_rows == 0)
  const uint32_t* row_ptr;    // nullable -> fixed_z nonzeros per row
  uint32_t n_rows, fixed_z;
  const uint32_t* csr_col;
  const float* csr_val;       // nullable -> binary features
  const float* y;             // labels in {-1,+1}
  int loss;                   // PSB_LOSS_*
  float* gcoef;               // out: d loss / d margin per row
  float* margin;              // out (nullable)
  double* stats;              // += {loss_sum, n_correct, n_rows}
  uint32_t* auc_hist;         // nullable: [2][4096] histogram of sigmoid(margin) by label
  uint32_t* bar;              // 2 words, grid barrier
  uint32_t* status;
} PsbPullParams;

// Worker half of a push (kernel F1a): X^T g over CSC segments, range partition,
// optional block-scaled quantisation, peer stores into the owners' inboxes, signal.
typedef struct {
  int S;
  uint32_t ts1;               // timestamp+1 published in the ready flags
  uint32_t inbox_cap;         // records per (owner, source) inbox
  int quant;                  // PSB_QUANT_*
  int send_keys;              // 0: values only (the owner reuses the slots of the previous push)
  const uint32_t* key_hit;    // nullable device flag with the same meaning, decided on the device
  uint32_t* mode[PSB_MAX_SHARDS];         // owner s's header word: 1 = keys omitted in this round
  psb_u64* inbox_keys[PSB_MAX_SHARDS];   // owner s's inbox for this source and ring slot
  void* inbox_vals[PSB_MAX_SHARDS];
  uint32_t* ready[PSB_MAX_SHARDS];        // owner s's ready flag for this source and ring slot
  uint32_t* count[PSB_MAX_SHARDS];        // owner s's record count word
  const uint32_t* applied[PSB_MAX_SHARDS];  // owner s's applied counter (ring reuse gate)
  uint32_t need_applied;
  const psb_u64* ukeys;
  const uint32_t* n_unique;
  const uint32_t* own_off;
  // gradient phase (skipped when nnz == 0: `grad` then holds user values)
  uint32_t nnz;
  const uint32_t* csc_row;
  const float* csc_val;       // nullable -> binary
  const uint32_t* flagbits;
  const uint32_t* wordbase;
  const float* gcoef;
  float* grad;                // per unique key; must be zero on entry when nnz > 0
  uint32_t* bar;              // 2 words
  uint32_t* done;             // 1 word, zero on entry, left zero
  uint32_t* status;
  // value width k (KVVector<K,V>(.., k), parameter/kv_vector.h:43-104): 0 or 1 = one value per key;
  // k > 1: `grad` holds k values per unique key (key-major) and nnz must be 0. The inbox then holds
  // count * k values per source, quantised in groups of 32 consecutive values.
  int width;
} PsbPushParams;

// Server half of a push (kernel F1b): wait for the sources' flags, reduce
// duplicate keys across sources, run the optimiser once per touched key.
typedef struct {
  int S;
  uint32_t ts1;
  uint32_t inbox_cap;
  int quant;
  void* table;
  psb_u64 mask;
  psb_u64 key_begin;
  psb_u64 slot_mult;
  const psb_u64* inbox_keys[PSB_MAX_SHARDS];
  const void* inbox_vals[PSB_MAX_SHARDS];
  const uint32_t* ready[PSB_MAX_SHARDS];
  const uint32_t* count[PSB_MAX_SHARDS];
  uint8_t alive[PSB_MAX_SHARDS];          // dead sources are skipped (their waits complete)
  uint8_t cached[PSB_MAX_SHARDS];         // key-cache hit: reuse slot_cache[r], no keys sent
  const uint32_t* mode[PSB_MAX_SHARDS];   // nullable: the source's header word (1 = keys omitted)
  uint32_t* slot_cache[PSB_MAX_SHARDS];   // per source: slot of each record (scratch + key cache)
  PsbOptimizer opt;
  double* stats;              // += {d_nnz, sum w^2, sum dw^2, n_updates}
  uint32_t* applied;          // set to ts1 when done
  uint32_t wait_iters;        // bounded wait budget for the ready flags (0 = default)
  uint32_t* bar;
  uint32_t* done;
  uint32_t* status;
  // value width k > 1 (sum entries only): the values live in wide_vals[slot * k + c], beside the table
  int width;
  float* wide_vals;
  // Several sources, every one with remembered slots: tile_off[r * (tiles + 1) + k] is the first record of
  // source r whose key lies in the k-th of `tiles` equal parts of this shard's key range (written by the
  // exchange pull of the same round). Records of one part from all sources are merged in shared memory
  // and every key gets one optimiser step and one entry write. Null: every record goes through the
  // accumulate-then-lead protocol. slow: one word, set while a part did not fit shared memory.
  const uint32_t* tile_off;
  int tiles;
  uint32_t* slow;
} PsbApplyParams;

// Two-sided pull fused with the margins (kernel F2, exchange form). One launch on
// every rank does three things: (a) store this worker's keys into the owners'
// request areas (coalesced peer stores, release flags); (b) as an owner, wait for
// each source's request, locate / insert the keys in the local table, remember
// the slots for the push of the same round, and store the weights straight into
// the requester's response buffer (coalesced peer stores, release flags); (c) as a
// worker again, wait for the owners' responses and compute margins, loss and
// d loss / d margin. Only bulk, coalesced traffic crosses NVLink.
typedef struct {
  int S;
  int me;
  uint32_t ts1;
  uint32_t need_applied;      // owner role: serve only after my shard applied this many rounds
  uint32_t req_cap;           // keys per (owner, source) request area
  uint32_t wait_iters;        // 0 = default budget
  int phases;                 // bit 0: (a), bit 1: (b), bit 2: (c); 7 = all in one launch. Separate
                              // launches exist for single-GPU emulation of several ranks, where a
                              // launch must never wait for a later launch.
  // (a) worker -> owners
  psb_u64* req_keys[PSB_MAX_SHARDS];     // owner s: request area of this source
  uint32_t* req_hdr[PSB_MAX_SHARDS];     // owner s: {count, base offset in my response buffer}
  uint32_t* req_ready[PSB_MAX_SHARDS];   // owner s: flag of this source
  // (b) owner role
  const psb_u64* my_req_keys[PSB_MAX_SHARDS];   // my request areas, one per source
  const uint32_t* my_req_hdr[PSB_MAX_SHARDS];
  const uint32_t* my_req_ready[PSB_MAX_SHARDS];
  float* resp_w[PSB_MAX_SHARDS];         // requester r: its response buffer
  uint32_t* resp_ready[PSB_MAX_SHARDS];  // requester r: flag of this owner
  uint32_t* slot_cache[PSB_MAX_SHARDS];  // per source: slot of every requested key (reused by the apply)
  uint8_t alive[PSB_MAX_SHARDS];
  void* table;
  psb_u64 mask, key_begin, slot_mult;
  const uint32_t* applied;               // my applied counter
  // (c) worker
  const float* my_resp_w;                // my response buffer (weights per unique key)
  const uint32_t* my_resp_ready[PSB_MAX_SHARDS];
  const psb_u64* ukeys;
  const uint32_t* n_unique;
  const uint32_t* own_off;
  float* grad_zero;
  const uint32_t* row_ptr;
  uint32_t n_rows, fixed_z;
  const uint32_t* csr_col;
  const float* csr_val;
  const float* y;
  int loss;
  float* gcoef;
  float* margin;
  double* stats;
  uint32_t* auc_hist;
  uint32_t* done;                        // 2 zeroed words
  uint32_t* status;
  // key-caching filter (filter/key_caching.h:9-60), decided inside the kernel: when this round's key
  // list is the previous round's (same fingerprint over every key and its position, same length),
  // phase (a) sends no keys and the owners answer from the slot lists they remembered.
  int key_cache;                         // 0 = off
  psb_u64* kc_state;                     // 4 words: {fingerprint, length + 1} of even and of odd rounds
  uint32_t* bar;                         // 2 zeroed words: grid barrier of the fingerprint pass
  const uint32_t* slot_cache_prev[PSB_MAX_SHARDS];   // owner role: the slot lists of the round before
  // value width k > 1: the owner answers with k values per key from wide_vals[slot * k + c]; the
  // response buffers hold k values per unique key (no margins in that case: n_rows must be 0)
  int width;
  const float* wide_vals;
  // nullable: where the owner notes, per source r, the first request of each of `tiles` (a power of two)
  // equal parts of its key range [key_begin, key_end) (key_end 0 = 2^64): tile_off[r * (tiles + 1) + k].
  // On a key-cache hit the previous round's notes (tile_off_prev) are copied.
  uint32_t* tile_off;
  const uint32_t* tile_off_prev;
  int tiles;
  psb_u64 key_end;
} PsbPullExchangeParams;

int psb_pull_exchange(const PsbPullExchangeParams* p, cudaStream_t stream);
int psb_table_init(void* table, psb_u64 capacity, cudaStream_t stream);
int psb_pull_margin(const PsbPullParams* p, cudaStream_t stream);
int psb_push(const PsbPushParams* p, cudaStream_t stream);
int psb_apply(const PsbApplyParams* p, cudaStream_t stream);
// Compacts (key, w) of every entry with w != 0 into out_keys/out_w; *out_n gets the count.
int psb_table_dump(const void* table, psb_u64 capacity, psb_u64* out_keys, float* out_w,
                   psb_u64 out_cap, unsigned long long* out_n, cudaStream_t stream);
// Bulk load (key, s0, s1, w) tuples into a table (checkpoint restore / model_input).
int psb_table_load(void* table, psb_u64 mask, psb_u64 key_begin, psb_u64 slot_mult, const psb_u64* keys, const float* s0,
                   const float* s1, const float* w, psb_u64 n, uint32_t* status,
                   cudaStream_t stream);
// Full state dump for checkpoints: every occupied slot.
int psb_table_export(const void* table, psb_u64 capacity, psb_u64* out_keys, float* out_s0,
                     float* out_s1, float* out_w, psb_u64 out_cap, unsigned long long* out_n,
                     cudaStream_t stream);

// number of CTAs a cooperative launch of the three fused kernels uses
int psb_coop_grid(int which);
int psb_struct_size(int which);   // 0 pull, 1 push, 2 apply, 3 optimizer, 4 pull exchange

// ---------------------------------------------------------------- filters / sorted-key utilities
int psb_key_signature(const psb_u64* keys, const uint32_t* n_ptr, uint32_t max_n, uint32_t* scratch,
                      uint32_t* state, uint32_t* hit, uint32_t* sig_out, cudaStream_t stream);
int psb_fixfloat_encode(const float* x, void* code, psb_u64 n, int nbytes, float lo, float hi, psb_u64 seed,
                        cudaStream_t stream);
int psb_fixfloat_decode(const void* code, float* x, psb_u64 n, int nbytes, float lo, float hi, cudaStream_t stream);
int psb_minmax(const float* x, psb_u64 n, float* out, cudaStream_t stream);
int psb_add_noise(float* x, psb_u64 n, float mean, float stdv, psb_u64 seed, cudaStream_t stream);
int psb_countmin_insert(uint32_t* cells, uint32_t n_cells, int k, const psb_u64* keys, const unsigned char* counts,
                        const uint32_t* n_ptr, uint32_t n, cudaStream_t stream);
int psb_countmin_query(const uint32_t* cells, uint32_t n_cells, int k, const psb_u64* keys, unsigned char* out,
                       const uint32_t* n_ptr, uint32_t n, cudaStream_t stream);
int psb_ordered_match(const psb_u64* src_key, const float* src_val, uint32_t n_src, const psb_u64* dst_key,
                      float* dst_val, uint32_t n_dst, int k, int op, unsigned long long* matched,
                      cudaStream_t stream);

// ---------------------------------------------------------------- Darlin block coordinate descent (F3)
// The model lives in a dense global column space (sorted union of all keys); shard s
// owns columns [shard_col[s], shard_col[s+1]). A worker's data is its rows in CSC
// order over its own unique keys (the output of sort + localise over the whole
// local data set); gcol maps a local unique key to its global column.
typedef struct {
  int S;
  uint32_t ts1;                 // block stamp + 1 (monotone)
  uint32_t c0, c1;              // global column range of the block
  uint32_t u0, u1;              // local unique-key range falling in the block
  uint32_t block_cap;           // capacity (columns) of the per-block exchange areas
  uint32_t shard_col[PSB_MAX_SHARDS + 1];
  // worker data
  const uint32_t* seg_off;      // CSC offsets over local unique keys
  const uint32_t* csc_row;
  const float* csc_val;         // nullable -> binary
  const uint32_t* flagbits;
  const uint32_t* wordbase;
  const uint32_t* gcol;         // local unique key -> global column
  const float* y;
  float* margin;                // X w per local row (the log-domain dual)
  const unsigned char* active;  // per global column (worker copy)
  const float* delta;           // trust region per global column (worker copy)
  float* stage;                 // [2][block_cap] local staging for (G, U)
  float* gu_inbox[PSB_MAX_SHARDS];   // owner s: [2][block_cap] area of this source
  uint32_t* ready[PSB_MAX_SHARDS];   // owner s: flag of this source
  uint32_t* bar; uint32_t* done; uint32_t* status;
  const uint32_t* csc_col;           // nullable: global column of every nonzero (saves two dependent gathers per nonzero)
  uint32_t nz0, nz1;                 // = seg_off[u0], seg_off[u1]: the block's nonzeros (filled by the host: one load level less)
} PsbDarlinGrad;

typedef struct {
  int S;
  uint32_t ts1;
  uint32_t c0, c1;              // block
  uint32_t my0, my1;            // my columns of the block (may be empty)
  uint32_t block_cap;
  const float* gu_inbox[PSB_MAX_SHARDS];   // my inbox areas, one per source
  const uint32_t* ready[PSB_MAX_SHARDS];
  uint8_t alive[PSB_MAX_SHARDS];
  float* w;                     // owner state per global column (only my range is used)
  float* delta;
  unsigned char* active;
  float eta, lambda, delta_max, kkt_threshold;
  float* wnew_inbox[PSB_MAX_SHARDS];       // dest r: [block_cap] new weights (NaN = deactivated)
  uint32_t* wnew_ready[PSB_MAX_SHARDS];    // dest r: flag of this owner
  float* violation;             // max |violation| (float as ordered int)
  uint32_t wait_iters;
  uint32_t* done; uint32_t* status;
} PsbDarlinUpdate;

typedef struct {
  int S;
  uint32_t ts1;
  uint32_t c0, c1, u0, u1;
  uint32_t block_cap;
  uint32_t shard_col[PSB_MAX_SHARDS + 1];
  const uint32_t* seg_off;
  const uint32_t* csc_row;
  const float* csc_val;
  const uint32_t* flagbits;
  const uint32_t* wordbase;
  const uint32_t* gcol;
  float* margin;
  float* w_cur;                 // worker copy of the weights per global column
  float* delta;
  unsigned char* active;
  float delta_max;
  const float* wnew;            // my wnew inbox [block_cap]
  const uint32_t* wnew_ready[PSB_MAX_SHARDS];  // flags of the owners
  uint8_t alive[PSB_MAX_SHARDS];
  uint32_t wait_iters;
  uint32_t* bar; uint32_t* status;
  const uint32_t* csc_col;           // nullable, as in PsbDarlinGrad
  uint32_t nz0, nz1;                 // as in PsbDarlinGrad
} PsbDarlinDual;

// A pass over n_steps feature blocks in one cooperative launch (see k_darlin_pass). grad / update /
// dual: device arrays of parameter blocks indexed [block * ring + stamp % ring], filled by the host
// (an update block with S == 0 means "no column of that block is mine"); order: device array of
// block indices; stamps ts_base .. ts_base + n_steps - 1.
typedef struct {
  const PsbDarlinGrad* grad;
  const PsbDarlinUpdate* update;
  const PsbDarlinDual* dual;
  const uint32_t* order;
  uint32_t n_steps;
  uint32_t ts_base;
  int tau;
  int ring;
  float kkt_threshold;
  uint32_t wait_iters;
  uint32_t* bar;
  uint32_t* status;
  psb_u64* phase_ns;            // optional: 4 accumulators of CTA 0's time per phase (see k_darlin_pass)
} PsbDarlinPass;
int psb_darlin_pass(const PsbDarlinPass* p, cudaStream_t stream);
int psb_darlin_grad(const PsbDarlinGrad* p, cudaStream_t stream);
int psb_darlin_update(const PsbDarlinUpdate* p, cudaStream_t stream);
int psb_darlin_dual(const PsbDarlinDual* p, cudaStream_t stream);
// out[0] += sum_rows log(1+exp(-y m)) ; out[1] += lambda*sum|w| over [c0,c1) ; out[2] += nnz(w) ; out[3] += #active
int psb_darlin_eval(const float* y, const float* margin, uint32_t n_rows, const float* w, const unsigned char* active,
                    uint32_t c0, uint32_t c1, float lambda, double* out, cudaStream_t stream);

// ---------------------------------------------------------------- data / misc
int psb_gen_batch(uint32_t* ids32, psb_u64* ids64, float* vals, float* y, uint32_t n_rows,
                  uint32_t z, psb_u64 n_feat, double zipf_s, psb_u64 seed, psb_u64 batch,
                  int real_values, cudaStream_t stream);
int psb_hash_ids(const uint32_t* ids32, const psb_u64* ids64, psb_u64* keys, psb_u64 n,
                 psb_u64 seed, cudaStream_t stream);
int psb_flush_l2(uint32_t* buf, psb_u64 n_words, uint32_t v, cudaStream_t stream);
// out[i] = bits [i * bits, (i + 1) * bits) of the little-endian word stream (which has a spare word at its end)
int psb_unpack_ids(const uint32_t* words, int bits, uint32_t n, uint32_t* out, cudaStream_t stream);
int psb_device_sm_count(void);

// ---------------------------------------------------------------- symmetric heap (CUDA IPC)
int psb_heap_alloc(void** ptr, size_t bytes);
int psb_heap_free(void* ptr);
int psb_ipc_export(void* ptr, void* handle_out /*64 host bytes*/);
int psb_ipc_open(const void* handle, void** ptr);
int psb_ipc_close(void* ptr);
int psb_ipc_handle_bytes(void);
int psb_set_device(int dev);
int psb_can_access_peer(int dev, int peer);
const char* psb_error_string(int neg_code);

#ifdef __cplusplus
}
#endif
