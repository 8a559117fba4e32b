// Host-callable launchers of every CUDA kernel in the extension.  This header is plain C++ (no
// torch, no device code) so the binding layer and the kernels compile independently.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rlk {
// Debug-bounds builds (-DRLK_DEBUG_BOUNDS=1): the error word that checked index accesses report to, per device.  The
// bindings register it; launchers read it (defined in runtime/runtime.cpp).
uint32_t* debug_error_word();
void bind_debug_error_word(int device, uint32_t* word);

// Kernel attributes such as the opt-in shared-memory size belong to one device's context.  A function-local
// ``static PerDeviceOnce flag;`` with ``if (flag.first()) { cudaFuncSetAttribute(...); }`` configures the kernel once
// on every device that launches it, not once per process.
struct PerDeviceOnce {
  bool done[64] = {};
  bool first() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return true;
    if (done[d]) return false;
    done[d] = true;
    return true;
  }
};
}  // namespace rlk

namespace rlk {

// ----------------------------------------------------------------------------- GEMM (tcgen05)
// D[M,N] = alpha * op(A) * op(B)^T (+ D if accumulate).
//   a_mn_major = false : A is row-major [M, K] (ld = lda);  true : A is row-major [K, M]
//   b_mn_major = false : B is row-major [N, K] (ld = ldb);  true : B is row-major [K, N]
// out_fp32 selects float (else bf16) output.  All leading dimensions are in elements; operand
// leading dimensions must be multiples of 8 and bases 16-byte aligned (TMA).
struct GemmArgs {
  const __nv_bfloat16* A;
  const __nv_bfloat16* B;
  void* D;
  int M, N, K;
  long long lda, ldb, ldd;
  bool a_mn_major, b_mn_major;
  bool out_fp32, accumulate;
  float alpha;
  int sm_count;
  uint32_t* err;
  // Grouped (mixture-of-experts) modes; rows of the token-side operand are grouped expert by expert and
  // every group's block is padded to a multiple of 128 rows.
  //   group_mode 1: D[M, N] = A[M, K] * B_g^T, g = tile_group[row / 128]; B stacks num_groups blocks.
  //   group_mode 2: D_g[M, N] = A[rows_g, M]^T * B[rows_g, N] with rows_g = group_offsets[g..g+1);
  //                 both operands MN-major, K = total rows, D stacks num_groups blocks of M rows, M % 128 == 0.
  int group_mode = 0;
  const int* tile_group = nullptr;
  const int* group_offsets = nullptr;
  int num_groups = 1;
  // Plain GEMM only: compute 256 x 256 tiles on pairs of SMs (tcgen05 cta_group::2, cluster of two CTAs).
  bool cta_pair = false;
};
void gemm_bf16(const GemmArgs& args, cudaStream_t stream);

// fp8 (e4m3) GEMM with one fp32 scale per row of A and per row of B: D[M, N] (bf16) = (A_q B_q^T) * sa[m] * sb[n].
// Operands are K-major codes with row pitches (bytes) that are multiples of 16.
void gemm_fp8_rowscaled(const void* a_q, long long lda, const float* scale_a, const void* b_q, long long ldb,
                        const float* scale_b, void* d, long long ldd, int M, int N, int K, bool cta_pair, int sm_count,
                        uint32_t* err, cudaStream_t stream);
// bf16 rows -> e4m3 codes and per-row scale (amax / 448); columns [cols, ldq) of the code rows are zero-filled.
void quantize_rows_e4m3(const void* x, long long ldx, long long rows, int cols, void* q, long long ldq, float* scale,
                        cudaStream_t stream);

// ----------------------------------------------------------------- fused linear -> log-prob
struct LinearLogpFwdArgs {
  const __nv_bfloat16* hidden;  // [n_tokens, hidden_dim]
  const __nv_bfloat16* weight;  // [v_local, hidden_dim]
  const long long* target;      // [n_tokens] global ids
  const float* bias;            // [v_local] or null
  int n_tokens, hidden_dim, v_local;
  long long ld_hidden, ld_weight;
  long long vocab_start;
  long long global_vocab;  // > 0: target ids outside [0, global_vocab) set kErrBadArgument (site 11) and give NaN
  int rank, world;
  int slot_base;      // first record slot of this rank in the partial buffers
  int total_records;  // records per row over all ranks (0: world * items_per_m)
  void* peer_partials[8];          // per rank: float4 [total_records, n_pad]
  unsigned int* peer_counters[8];  // per rank: [tiles_m] counters of the set used by this launch
  unsigned int* next_counters;     // local: the set the next launch will use (zeroed here)
  int counter_capacity;            // entries per counter set
  float* logp;
  float* lse;
  float* entropy;
  int sm_count;
  uint32_t* err;
  unsigned long long wait_limit_ns;  // 0 = default
};
void linear_logp_forward(const LinearLogpFwdArgs& args, cudaStream_t stream);
void linear_logp_workspace_shape(int n_tokens, int v_local, int world, int* items_per_m, int* n_pad, int* tiles_m);

struct LinearLogpDzArgs {
  const __nv_bfloat16* hidden;
  const __nv_bfloat16* weight;
  const long long* target;
  const float* bias;
  const float* lse;
  const float* grad;
  int n_tokens, hidden_dim, v_local;
  long long ld_hidden, ld_weight;
  long long vocab_start;
  __nv_bfloat16* dz;
  long long ld_dz;
  int sm_count;
  uint32_t* err;
};
void linear_logp_dz(const LinearLogpDzArgs& args, cudaStream_t stream);

}  // namespace rlk

namespace rlk {

// dtype codes used by the elementwise / row kernels: 0 = float32, 1 = bfloat16, 2 = float16.

// ------------------------------------------------------------------ log-prob over logits rows
struct LogpRowsArgs {
  const void* logits;  // [rows, V] with row pitch ld (elements)
  long long ld;
  int in_dtype;
  const long long* ids;          // [rows]
  const long long* row_indices;  // [launch_rows] or null (dense)
  int launch_rows;
  int V;
  void* out;  // [rows]
  int out_dtype;
  long long total_rows;  // rows of ``logits`` (0: unknown); gathered row indices are checked against it in debug builds
};
void logp_rows(const LogpRowsArgs& args, cudaStream_t stream);

struct RatioKlFwdArgs {
  const void* policy;
  const void* ref;  // null: reference == policy
  long long ld_policy, ld_ref;
  int dtype;
  const long long* ids;
  const unsigned char* mask;
  const float* old_logp;
  int rows, V;
  float* ratio;
  float* kl;
  float* save_d;
  float* save_lse;
  float* save_lp;  // policy log-prob of the selected token
  unsigned int* bad_id_flag;
};
void ratio_kl_forward(const RatioKlFwdArgs& args, cudaStream_t stream);

struct RatioKlBwdArgs {
  const void* policy;
  long long ld_policy;
  int dtype;
  const long long* ids;
  const unsigned char* mask;
  const float* g_ratio;
  const float* g_kl;
  const float* ratio;
  const float* save_d;
  const float* save_lse;
  int rows, V;
  void* grad;
  long long ld_grad;
};
void ratio_kl_backward(const RatioKlBwdArgs& args, cudaStream_t stream);

}  // namespace rlk

namespace rlk {

// -------------------------------------------------------------------------------- RL losses
// bounds == null -> uniform groups of `uniform` sequences.
// n_rewards: length of ``rewards`` / ``adv`` (group bounds are checked against it in debug-bounds builds)
void group_advantages(const float* rewards, const long long* bounds, int num_groups, long long uniform, float eps,
                      float* adv, long long n_rewards, cudaStream_t stream);

struct SurrogateFwdArgs {
  const float* logp;      // [n] policy log-probs
  const float* ref_logp;  // [n] or null (kl = 0)
  const float* old_logp;  // [n]
  const float* adv_seq;   // [n / T] per-sequence advantages, or null
  const float* adv_tok;   // [n] per-token advantages, or null
  const unsigned char* mask;
  long long n, T;
  float clip_eps, beta;
  float* d_pl;       // [n] unit gradient of the policy term
  float* d_kl;       // [n] unit gradient of the kl term
  float* ratio_out;  // [n] or null
  float* kl_out;     // [n] or null
  float* partials;   // [surrogate_partial_floats()]
  float* out4;       // {loss, policy_loss, kl, active count}
};
int surrogate_partial_floats();
void surrogate_forward(const SurrogateFwdArgs& args, cudaStream_t stream);
void surrogate_backward(const float* d_pl, const float* d_kl, const float* stats, const float* g3, float beta,
                        long long n, float* grad_logp, cudaStream_t stream);
void dpo_forward(const float* pc, const float* pr, const float* rc, const float* rr, int n, float beta, float ls,
                 float* out_loss, float* chosen_reward, float* rejected_reward, float* dh, cudaStream_t stream);

}  // namespace rlk

namespace rlk {

// --------------------------------------------------------------------------- model-side ops
void rmsnorm_forward(const void* x, long long ldx, int x_dtype, const void* w, int w_dtype, void* y, long long ldy,
                     bool out_fp32, long long rows, int D, float eps, float* rstd, cudaStream_t stream);
// Rows that one CTA of the backward kernel walks (a function of the row count only) and the number of CTAs =
// rows of the partial-sum scratch ``dw_part [chunks, D]``.  rows_per_cta <= 0 selects the default for ``rows``.
int rmsnorm_bwd_rows_per_cta(long long rows);
int rmsnorm_bwd_chunks(long long rows, int rows_per_cta = 0);
void rmsnorm_backward(const void* x, long long ldx, int x_dtype, const void* w, int w_dtype, const void* dy,
                      long long lddy, const float* rstd, void* dx, long long lddx, long long rows, int D,
                      float* dw_part, void* dw, cudaStream_t stream, int rows_per_cta = 0);
// Per-head RMSNorm (head_dim 128) of the q and k heads inside a packed qkv buffer [tokens, (hq + 2 hkv) * 128]; v is copied.
// Backward writes per-block partial weight gradients ``part [qk_norm_blocks(...)][2][128]`` (q, then k).
int qk_norm_blocks(long long tokens, int heads);
void qk_norm_forward(const __nv_bfloat16* qkv, long long ld, __nv_bfloat16* out, long long ldo, const __nv_bfloat16* wq,
                     const __nv_bfloat16* wk, long long tokens, int hq, int hkv, float eps, cudaStream_t stream);
void qk_norm_backward(const __nv_bfloat16* qkv, long long ld, const __nv_bfloat16* dout, long long ldg,
                      __nv_bfloat16* dqkv, long long ldd, const __nv_bfloat16* wq, const __nv_bfloat16* wk,
                      long long tokens, int hq, int hkv, float eps, float* part, cudaStream_t stream);
// up == null -> plain SiLU
void swiglu_forward(const void* gate, long long ldg, const void* up, long long ldu, int dtype, void* out, long long ldo,
                    bool out_fp32, long long rows, int F, cudaStream_t stream);
void swiglu_backward(const void* gate, long long ldg, const void* up, long long ldu, const void* dy, long long lddy,
                     int dtype, void* dgate, long long lddg, void* dup, long long lddu, long long rows, int F,
                     cudaStream_t stream);
// packed bf16 [gate | up] rows of width 2F; dgu receives [dgate | dup]
void swiglu_packed_forward(const __nv_bfloat16* gu, long long ldgu, __nv_bfloat16* out, long long ldo, long long rows, int F,
                           cudaStream_t stream);
void swiglu_packed_backward(const __nv_bfloat16* gu, long long ldgu, const __nv_bfloat16* dy, long long lddy,
                            __nv_bfloat16* dgu, long long lddgu, long long rows, int F, cudaStream_t stream);
// out[n, Hkv * rep * 128] = merge by log-sum-exp of two partial attention results o1 / o2 [n * rep, Hkv, 128] (bf16)
// with l1 / l2 [Hkv, n * rep]; rows = n * rep.
void attn_merge2(const void* o1, const float* l1, const void* o2, const float* l2, void* out, long long rows, int hkv,
                 int rep, cudaStream_t stream);
// table_rows: rows of the cos / sin tables (positions are checked against it in debug-bounds builds)
void rope_apply(const void* x, long long ldt, int dtype, const long long* pos, const float* cos_t, const float* sin_t,
                void* out, long long ldo, long long tokens, int heads, int D, bool inverse, long long table_rows,
                cudaStream_t stream);
void embedding_forward(const long long* ids, const void* table, long long ldw, int dtype, void* out, long long rows,
                       int D, long long vocab, cudaStream_t stream);
void embedding_backward(const long long* seg_ids, const long long* seg_start, long long segments,
                        const long long* order, const void* dy, int dy_dtype, int D, void* dtable, bool table_fp32,
                        long long ldw, long long dy_rows, long long table_rows, cudaStream_t stream);
// master: fp32 master weights or nullptr.  residual: 16-bit residuals of a bf16 parameter (fp32 master = parameter
// bits << 16 plus the sign-extended residual) or nullptr; at most one of the two.
void adamw_step(void* p, int p_dtype, float* master, short* residual, const void* g, int g_dtype, float* m, float* v,
                long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
                cudaStream_t stream);

}  // namespace rlk

namespace rlk {

// ---------------------------------------------------------------------------------- sampler
// top_k in [1, sample_topk_limit()], top_p in (0, 1] (1 disables the nucleus cut).
void sample_topk_topp(const void* logits, long long ld, int dtype, int rows, int V, int top_k, float top_p,
                      float temperature, unsigned long long seed, unsigned long long offset, long long* out_ids,
                      float* out_logprob, cudaStream_t stream);
int sample_topk_limit();
// Full-vocabulary nucleus (top-p only) / plain temperature sampling (top_p = 1).
void sample_nucleus(const void* logits, long long ld, int dtype, int rows, int V, float top_p, float temperature,
                    unsigned long long seed, unsigned long long offset, long long* out_ids, float* out_logprob,
                    cudaStream_t stream);

}  // namespace rlk

namespace rlk {

// -------------------------------------------------------------------------------- attention
// Packed-token attention with head_dim 128.  `seqs` holds 8 int32 per sequence:
//   {q_start, q_len, prefix_k_start, prefix_k_len, self_k_start, self_k_len, 0, 0}
// `tiles` holds (sequence, first query row in that sequence) per 128-row query tile.
struct AttnFwdArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  long long ld_q, ld_k, ld_v;  // token pitches (elements)
  long long total_q, total_kv;
  int heads_q, heads_kv;
  const int* seqs;
  int num_seqs;  // rows of ``seqs`` (layout tables are checked against it and the token counts in debug-bounds builds)
  const int* tiles;
  int num_tiles;
  bool causal;
  float softmax_scale;
  __nv_bfloat16* out;
  long long ld_out;
  float* lse;  // [heads_q, total_q] or null
  long long lse_head_stride;
  uint32_t* err;
  int sm_count = 148;  // CTAs of the persistent grid
};
void attention_forward(const AttnFwdArgs& args, cudaStream_t stream);

}  // namespace rlk

namespace rlk {

// ----------------------------------------------------------------------- attention backward
// kv_items: 8 int32 each {k_row, k_len, k_pos, qb_begin, qb_end, out_slot, 0, 0}
// q_blocks: 4 int32 each {q_row, n_rows, q_pos, causal};  reduce_jobs: 4 int32 {k_row, k_len, slot_begin, slot_end}
struct AttnBwdArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* dout;
  long long ld_q, ld_k, ld_v, ld_do;
  long long total_q, total_kv;
  int heads_q, heads_kv;
  const int* seqs;
  const int* q_tiles;
  int num_q_tiles;
  const int* kv_items;
  int num_kv_items;
  const int* q_blocks;
  const int* reduce_jobs;
  int num_reduce_jobs;
  bool causal;
  float softmax_scale;
  const float* lse;    // [heads_q, total_q]
  const float* delta;  // [heads_q, total_q]
  __nv_bfloat16* dq;
  long long ld_dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long ld_dkv;
  float* partials;  // [slots, heads_kv, 2, 128, 128]
  uint32_t* err;
};
void attention_delta(const __nv_bfloat16* out, const __nv_bfloat16* dout, long long ld, int heads, long long tokens,
                     float* delta, cudaStream_t stream);
void attention_backward_dq(const AttnBwdArgs& args, cudaStream_t stream);
void attention_backward_dkv(const AttnBwdArgs& args, cudaStream_t stream);

}  // namespace rlk

namespace rlk {

// ------------------------------------------------------------ peer-memory communication kernels
void peer_barrier(void* const* pads, int rank, int world, unsigned int epoch, unsigned long long limit_ns, uint32_t* err,
                  cudaStream_t stream);
// skip_if_set: error word of the preceding device barrier (the kernel applies nothing if it is non-zero) or nullptr;
// max_blocks > 0 limits the grid, for launches that share the GPU with compute on another stream.
void zero1_fused_step(void* const* grads, void* const* params, int rank, int world, long long lo, long long hi, float* m,
                      float* v, float* master, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                      float grad_scale, const uint32_t* skip_if_set, int max_blocks, cudaStream_t stream);
void peer_sum(void* const* srcs, int world, long long n, bool src_fp32, void* out, bool out_fp32, cudaStream_t stream);
// 64-bit position-weighted digest of ``nbytes`` bytes at ``data`` (16-byte aligned), added into *out.
void weight_digest64(const void* data, long long nbytes, unsigned long long* out, cudaStream_t stream);
// Many tensors in one launch.  ``table``: device rows of four int64 (source address, destination byte offset or result
// slot, elements or bytes, units of all earlier rows), a unit being 32768 elements (cast) or 64-bit words (digest).
void cast_segments(const void* table, int count, long long total_units, int src_dtype, int dst_dtype, void* dst_base,
                   cudaStream_t stream);
void digest_segments(const void* table, int count, long long total_units, unsigned long long* results, cudaStream_t stream);
void cast_broadcast(const void* src, int src_dtype, void* const* dsts, int dst_dtype, int world, long long n,
                    cudaStream_t stream);

}  // namespace rlk

namespace rlk {

// ---------------------------------------------------------------------------- mixture of experts
// experts <= 512, k <= 32; hidden % 8 == 0 and 16-byte aligned rows for the row kernels.
void moe_topk(const float* logits, int tokens, int experts, int k, int* idx, float* weight, cudaStream_t stream);
void moe_topk_backward(const int* idx, const float* weight, const float* dweight, int tokens, int experts, int k,
                       float* dlogits, cudaStream_t stream);
void moe_gather_rows(const __nv_bfloat16* src, long long ld_src, const int* src_row, const float* scale,
                     __nv_bfloat16* dst, long long ld_dst, int slots, int hidden, cudaStream_t stream,
                     long long src_rows = 0, uint32_t* err = nullptr);  // last two: checked indexing in debug builds
void moe_combine(const __nv_bfloat16* src, long long ld_src, const int* slot, const float* weight, int k,
                 __nv_bfloat16* out, long long ld_out, int tokens, int hidden, cudaStream_t stream,
                 long long src_rows = 0, uint32_t* err = nullptr);
void moe_rowdot(const __nv_bfloat16* a, long long ld_a, const __nv_bfloat16* b, long long ld_b, const int* slot, int k,
                int tokens, int hidden, float* out, cudaStream_t stream);
#ifdef RLK_ATTN_PROFILE
void attention_profile_read(unsigned long long* out);
void attention_profile_reset();
void attention_bwd_profile_read(unsigned long long* out);
#endif

// ---- tracing (trace.cu): out[slot] = %globaltimer in stream order
void device_stamp(unsigned long long* out, int slot, cudaStream_t stream);

// ---- tensor-parallel linears fused with their collectives (tp_linear.cu) -------------------------
struct TpAgGemmArgs {
  const __nv_bfloat16* x_local;  // [rows_local, K] this rank's rows
  long long ldx;
  int rows_local;                // multiple of 128
  int K, N;
  const __nv_bfloat16* B;        // [N, K] (K-major) or [K, N] (b_mn)
  long long ldb;
  bool b_mn;
  __nv_bfloat16* C;              // [rows_local * world, N]
  long long ldc;
  int rank, world;
  unsigned int epoch;            // 1, 2, ... per use of this buffer set
  int chunks;                    // column chunks per tile (arrivals per tile and call)
  void* gathered[8];             // bf16 [M, K] on every rank
  void* ready[8];                // unsigned int [M / 128] on every rank
  unsigned long long wait_ns;
  int sm_count;
  uint32_t* err;
};
void tp_ag_gemm(const TpAgGemmArgs& a, cudaStream_t stream);

struct TpGemmRsArgs {
  const __nv_bfloat16* A;        // [rows_local * world, K]
  long long lda;
  int rows_local;                // multiple of 128
  int K, N;
  const __nv_bfloat16* B;
  long long ldb;
  bool b_mn;
  __nv_bfloat16* out;            // [rows_local, N]
  long long ldo;
  int rank, world;
  unsigned int target;           // world * (uses of this buffer set so far, this one included)
  void* partial[8];              // bf16 [world, rows_local, N] on every rank
  void* counters[8];             // unsigned int [rows_local / 128 * ceil(N / 256)] on every rank
  unsigned long long wait_ns;
  int sm_count;
  uint32_t* err;
};
void tp_gemm_rs(const TpGemmRsArgs& a, cudaStream_t stream);

// Dispatch plan on the device: slot of every assignment, token of every slot (src_row must be pre-filled with -1),
// expert of every 128-row tile, padded expert offsets [E + 1] and counts [E].  chunk_hist: scratch [ceil(A / 256), E].
void moe_build_plan(const int* idx, int assignments, int k, int experts, int num_slots, int unused_group, int* chunk_hist,
                    int* offsets, int* counts, int* tile_group, int* slot, int* src_row, cudaStream_t stream);
// expert parallelism over peer-mapped buffers (dst / src / b hold one base pointer per rank)
void moe_scatter_rows_peer(const __nv_bfloat16* src, long long ld_src, const int* token, const int* dest_rank,
                           const int* dest_slot, const float* scale, void* const* dst, int world, long long ld_dst,
                           int assignments, int hidden, cudaStream_t stream);
void moe_combine_peer(void* const* src, int world, long long ld_src, const int* rank, const int* slot, const float* weight,
                      int k, __nv_bfloat16* out, long long ld_out, int tokens, int hidden, cudaStream_t stream);

}  // namespace rlk
