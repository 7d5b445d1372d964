/*
 * mxk -- sequence-mixing kernels for NVIDIA B200 (sm_100a) behind a plain C ABI.
 *
 * Every function below replaces one computation that memorax performs with
 * jax.lax.associative_scan inside Memoroid.scan_fn
 * (memorax/networks/sequence_models/memoroid.py:60-91) plus the cell-specific
 * operator / read-out named in its comment.  The reference has no FFI of its
 * own; these are the entry points an XLA custom call (jax.ffi) or any other
 * host would bind.
 *
 * Conventions
 *   - Launch-only: each call validates its arguments on the host, enqueues
 *     kernels on `stream` and returns.  No host synchronisation, no allocation,
 *     no retained pointers.  All buffers, outputs and workspaces included, are
 *     device memory owned by the caller.  The one exception is
 *     mxk_linrec_c64_bwd_noalloc, which keeps its scratch in the library's own
 *     device image and remembers that array's address per device (see there).
 *   - Layout: batch-major, time second, features last, C-contiguous --
 *     (B, T, D) or (B, T, H, d); `done` is (B, T) bytes, non-zero = "step t is
 *     the first step of a new episode", i.e. the state before step t is
 *     discarded (memoroid.py:67-85).  `done` may be NULL (no resets).
 *     Contiguity is part of the contract: there are no stride arguments, a host
 *     that holds a strided view copies it first (XLA hands custom calls dense
 *     row-major buffers, so the jax.ffi binding never has to).
 *   - Carries are passed without the reference's singleton time axis:
 *     (B, D) or (B, H, dv, dk).
 *   - Complex tensors are interleaved (re, im) float pairs.  Complex
 *     cotangents follow JAX's convention (no conjugation anywhere), which is
 *     the conjugate of torch.autograd's.
 *   - Return value: 0 = enqueued; negative = argument rejected before any
 *     launch (MXK_ERR_*); positive = cudaError_t reported by the launch.
 */
#ifndef MXK_H_
#define MXK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* mxk_stream_t; /* a cudaStream_t / CUstream */

enum {
  MXK_OK = 0,
  MXK_ERR_NULL = -1,        /* a required pointer is NULL */
  MXK_ERR_DIMS = -2,        /* a dimension is non-positive or too large */
  MXK_ERR_ALIGN = -3,       /* a pointer is not 16-byte aligned */
  MXK_ERR_UNSUPPORTED = -4, /* head dim / chunk size outside the compiled set */
  MXK_ERR_WORKSPACE = -5,   /* workspace missing or too small */
  MXK_ERR_SCRATCH_LIMIT = -6 /* problem larger than the library's built-in scratch buffer */
};

/* Human-readable text for a status returned by any function below. */
const char* mxk_status_string(int status);
/* ABI version of the loaded library (bumped on signature changes). */
int mxk_abi_version(void);

/* Failure-path self-test.  Every tensor-core kernel below waits for its copies
 * and MMAs with a bounded poll and, when a wait gives up, sets the caller's
 * `status` word to 1 and drains instead of spinning or trapping.  This launches
 * a one-thread kernel that waits, with the same primitive and a limit of
 * `polls` (1..16, about a millisecond each), on a barrier that nothing ever
 * completes, so a host can check that the word really gets set and that the
 * context survives.  It has no counterpart in the reference.
 *   status  device int, expected to read 1 after the stream has drained */
int mxk_selftest_bounded_wait(int* status, int polls, mxk_stream_t stream);

/* ---------------------------------------------------------------------------
 * Diagonal linear recurrence  h_t = done_t ? b_t : a_t * h_{t-1} + b_t
 * with the decay leaf          A_t = done_t ? a_t : a_t * A_{t-1}.
 *
 * Replaces Memoroid.scan_fn over the (state, decay) operator of
 * lru.py:92-95 / s5.py:133-136 / mamba.py:119-122 (decay broadcast over the
 * state_dim x head_dim elements of a head) and the multiplicative-reset scan
 * of memoroid.py:114-141.
 *
 *   a       (B,T,D), or (D) when a_time_invariant != 0 (lru.py:86)
 *   b       (B,T,D)
 *   h0      (B,D) carried state, NULL = zeros (lru.py:104-108)
 *   a0      (B,D) carried decay leaf, NULL = ones; read only if a_last != NULL
 *   h       (B,T,D) out: every state (next carry's state is h[:, T-1])
 *   a_last  (B,D) out, optional: decay leaf of the next carry (memoroid.py:89)
 * f32: real floats.  c64: complex64, D counts complex elements.
 * ------------------------------------------------------------------------- */
int mxk_linrec_f32_fwd(const float* a, int a_time_invariant, const float* b, const float* h0,
                       const float* a0, const uint8_t* done, float* h, float* a_last,
                       int B, int T, int D, mxk_stream_t stream);
int mxk_linrec_c64_fwd(const float* a, int a_time_invariant, const float* b, const float* h0,
                       const float* a0, const uint8_t* done, float* h, float* a_last,
                       int B, int T, int D, mxk_stream_t stream);

/* Reverse-mode of the above (what jax.grad derives from the scan; the
 * reference has no hand-written rule).  With m_t = !done_t and
 * g_t = gh_t + a_{t+1} m_{t+1} g_{t+1}   (gh_last is added to gh_{T-1}):
 *   gb_t = g_t;  ga_t = m_t h_{t-1} g_t;  gh0 = a_1 m_1 g_1.
 *
 *   h        (B,T,D) states saved by the forward call;  h0 as in forward
 *   gh       (B,T,D) cotangent of h;  gh_last (B,D) cotangent of the carried
 *            state, NULL = zeros
 *   gb       (B,T,D) out
 *   ga       out, optional: (B,T,D), or (D) summed over batch and time when
 *            a_time_invariant (needs `workspace`)
 *   gh0      (B,D) out, optional
 *   workspace  scratch of mxk_linrec_bwd_workspace_bytes(...) bytes, only for
 *            the time-invariant ga reduction; contents undefined afterwards.
 * The decay leaf a_last has no cotangent (every read-out ignores it). */
size_t mxk_linrec_bwd_workspace_bytes(int is_complex, int a_time_invariant, int B, int T, int D);
int mxk_linrec_f32_bwd(const float* a, int a_time_invariant, const float* h, const float* h0,
                       const uint8_t* done, const float* gh, const float* gh_last, float* gb,
                       float* ga, float* gh0, void* workspace, size_t workspace_bytes,
                       int B, int T, int D, mxk_stream_t stream);
/* c64 only: `conjugate` != 0 runs the same recurrences with conj(a) and
 * conj(h), which maps torch.autograd-convention cotangents in to
 * torch-convention cotangents out without separate conjugation passes;
 * 0 = JAX convention. */
int mxk_linrec_c64_bwd(const float* a, int a_time_invariant, const float* h, const float* h0,
                       const uint8_t* done, const float* gh, const float* gh_last, float* gb,
                       float* ga, float* gh0, void* workspace, size_t workspace_bytes,
                       int B, int T, int D, int conjugate, mxk_stream_t stream);

/* State after the LAST step only, h_T (B,D), of the same recurrences: nothing is stored per step, so the launch is
 * one read stream.  This is what Memoroid._propagate_sensitivities returns per parameter leaf (memoroid.py:114-141:
 * the scan's last element, `x[:, -1:]`); the reference materialises all T steps to take it. */
int mxk_linrec_f32_last(const float* a, int a_time_invariant, const float* b, const float* h0, const uint8_t* done,
                        float* h_last, int B, int T, int D, mxk_stream_t stream);
int mxk_linrec_c64_last(const float* a, int a_time_invariant, const float* b, const float* h0, const uint8_t* done,
                        float* h_last, int B, int T, int D, mxk_stream_t stream);

/* The real recurrence with one decay per GROUP of channels: a is (B,T,G), D = G * group channels,
 * channel c uses a[..., c / group].  This is MambaCell's scan (mamba.py:109-122: a scalar decay per
 * (b, t, head) over a state_dim x head_dim matrix state) without expanding the decay to full width.
 * group must be a multiple of 128 (MXK_ERR_UNSUPPORTED otherwise: expand the decay and use
 * mxk_linrec_f32_fwd).  a0 / a_last, the decay leaf of the carry, are (B,G).
 * Backward: ga (B,T,G) is reduced over each group in the kernel (fixed order, no atomics);
 * `workspace` of mxk_linrec_grouped_bwd_workspace_bytes(...) bytes is needed when group > 128. */
size_t mxk_linrec_grouped_bwd_workspace_bytes(int B, int T, int D, int G);
int mxk_linrec_f32_grouped_fwd(const float* a, const float* b, const float* h0, const float* a0, const uint8_t* done,
                               float* h, float* a_last, int B, int T, int D, int G, mxk_stream_t stream);
/* h_T (B,D) only, as mxk_linrec_f32_last. */
int mxk_linrec_f32_grouped_last(const float* a, const float* b, const float* h0, const uint8_t* done, float* h_last,
                                int B, int T, int D, int G, mxk_stream_t stream);
int mxk_linrec_f32_grouped_bwd(const float* a, const float* h, const float* h0, const uint8_t* done, const float* gh,
                               const float* gh_last, float* gb, float* ga, float* gh0, void* workspace,
                               size_t workspace_bytes, int B, int T, int D, int G, mxk_stream_t stream);

/* Allocation-free variant of mxk_linrec_c64_bwd for a time-invariant decay
 * (the LRU / S5 case).  It has no counterpart in the reference; it exists for
 * hosts that cannot hand this library a workspace.  An XLA custom call is
 * given exactly the operand and result buffers the compiler planned at trace
 * time, a CUDA-graph replay cannot grow a buffer, and an acting loop that steps
 * environments every few hundred microseconds cannot afford cudaMalloc's
 * device-wide synchronisation -- yet the (D,) decay gradient needs B * D
 * partial sums somewhere.  Here they go into a fixed 4 MiB array that lives in
 * the library's device image (every GPU that loads the library holds it until
 * the process exits), so the caller passes inputs and outputs only.
 *
 *   - Limit: B * D <= mxk_linrec_noalloc_max_elements() (524288 complex
 *     elements); larger problems return MXK_ERR_SCRATCH_LIMIT and launch nothing.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, no allocation); make that first call before any
 *     stream capture begins.  The address is remembered per device ordinal for
 *     the life of the process: after cudaDeviceReset (or any teardown of the
 *     device's primary context) it is stale, so a process that resets a device
 *     must not call this function on it again.
 *   - All calls on a device share the one array.  Every partial sum is
 *     overwritten before it is read, so nothing has to be cleared between
 *     calls, but two calls whose kernels overlap on the GPU (different streams)
 *     race on it: serialise them.
 * Arguments as mxk_linrec_c64_bwd with a_time_invariant = 1; `ga` is (D). */
size_t mxk_linrec_noalloc_max_elements(void);
int mxk_linrec_c64_bwd_noalloc(const float* a, const float* h, const float* h0, const uint8_t* done,
                               const float* gh, const float* gh_last, float* gb, float* ga, float* gh0,
                               int B, int T, int D, int conjugate, mxk_stream_t stream);

/* ---------------------------------------------------------------------------
 * Log-space recurrence (MinGRU, min_gru.py:67-78):
 *   x_t = done_t ? ls_t : logaddexp(d_t + x_{t-1}, ls_t)
 *   A_t = done_t ? d_t  : d_t + A_{t-1}
 * x0 may hold -inf (min_gru.py:80-90); NULL = -inf.  a0 NULL = zeros.
 *   x  (B,T,D) out: log states;  y (B,T,D) out, optional: exp(x), the read-out.
 * Backward: gx is the cotangent of x, gy (optional) that of y; with
 * w_t = m_t exp(d_t + x_{t-1} - x_t) and G_t = gx_t + gy_t y_t + w_{t+1} G_{t+1}:
 *   gls_t = (1 - w_t) G_t;  gd_t = w_t G_t;  gx0 = w_1 G_1.
 * ------------------------------------------------------------------------- */
int mxk_loglinrec_f32_fwd(const float* ls, const float* d, const float* x0, const float* a0,
                          const uint8_t* done, float* x, float* y, float* a_last,
                          int B, int T, int D, mxk_stream_t stream);
int mxk_loglinrec_f32_bwd(const float* d, const float* x, const float* x0, const uint8_t* done,
                          const float* gx, const float* gy, const float* gx_last, float* gls,
                          float* gd, float* gx0, int B, int T, int D, mxk_stream_t stream);

/* The same recurrence with MinGRU's gate math fused in (min_gru.py:52-61): the kernels take the two Dense
 * layers' pre-activations z and h~ (B,T,D) and form the elements on the fly,
 *   log_state = -softplus(-z) + log g(h~),  decay = -softplus(z),  g(h) = h >= 0 ? h + 0.5 : sigmoid(h),
 * so the (B,T,D) log_state and decay tensors are never written or read back.  Backward returns the
 * cotangents of z and h~ (gz, gh).  Other arguments as mxk_loglinrec_f32_fwd / _bwd. */
int mxk_mingru_f32_fwd(const float* z, const float* h_tilde, const float* x0, const float* a0, const uint8_t* done,
                       float* x, float* y, float* a_last, int B, int T, int D, mxk_stream_t stream);
int mxk_mingru_f32_bwd(const float* z, const float* h_tilde, const float* x, const float* x0, const uint8_t* done,
                       const float* gx, const float* gy, const float* gx_last, float* gz, float* gh, float* gx0,
                       int B, int T, int D, mxk_stream_t stream);

/* ---------------------------------------------------------------------------
 * Chunked causal linear attention with carried state (linear_attention.py:58-124
 * under Memoroid.scan_fn): per head, S_t = [!done_t] S_{t-1} + v_t phi(k_t)^T,
 * z_t = [!done_t] z_{t-1} + phi(k_t), o_t = S_t phi(q_t) / max(phi(q_t).z_t, eps),
 * phi = elu + 1 when feature_map != 0 (else q, k are used as given).
 * The reference materialises every S_t; here the state is carried chunk to
 * chunk (64 tokens) in fp32 and only (B,H,d,d) ever touches memory.
 *
 *   q, k, v   (B,T,H,d) bf16, contiguous;  d a multiple of 8, at most 64 (else MXK_ERR_UNSUPPORTED).
 *             The kernels work on 64-column tiles; for d < 64 the tensor maps zero-fill the
 *             columns past d on loads and clip them on stores.
 *   s0        (B,H,d_v,d_k) fp32 carried S, NULL = zeros;  z0 (B,H,d_k), NULL = zeros
 *   o         (B,T,H,d) bf16 out
 *   s_last, z_last   next carry, optional
 *   chunk_states  optional residual for the backward call,
 *             mxk_linattn_chunk_states_bytes(...) bytes: the bf16 state entering
 *             every chunk in tensor-core operand order
 *   status    optional device int, set non-zero if a bounded device-side wait
 *             gave up (results are then undefined)
 * ------------------------------------------------------------------------- */
size_t mxk_linattn_chunk_states_bytes(int B, int T, int H, int d);
int mxk_linattn_bf16_fwd(const void* q, const void* k, const void* v, const float* s0, const float* z0,
                         const uint8_t* done, void* o, float* s_last, float* z_last, void* chunk_states,
                         int* status, int B, int T, int H, int d, float eps, int feature_map,
                         mxk_stream_t stream);

/* Reverse mode of mxk_linattn_bf16_fwd (what jax.grad derives from the scan and
 * read-out; the clamp max(den, eps) passes no gradient where it is active).
 *   d_o       (B,T,H,d) bf16 cotangent of o
 *   chunk_states  the residual written by the forward call on the same inputs
 *   ds_last, dz_last  cotangents of the next carry, NULL = zeros
 *   dq, dk, dv  (B,T,H,d) bf16 out;  ds0 (B,H,d,d), dz0 (B,H,d) fp32 out, optional
 * `done` has no cotangent. */
int mxk_linattn_bf16_bwd(const void* q, const void* k, const void* v, const void* d_o, const void* chunk_states,
                         const uint8_t* done, const float* ds_last, const float* dz_last, void* dq, void* dk,
                         void* dv, float* ds0, float* dz0, int* status, int B, int T, int H, int d, float eps,
                         int feature_map, mxk_stream_t stream);

/* ---------------------------------------------------------------------------
 * mLSTM, the matrix-memory LSTM (mlstm.py:163-240 under Memoroid.scan_fn): per head,
 * with the running-max stabiliser m of the reference's operator (mlstm.py:205-229),
 *   m_t = max(m_{t-1} + log_f_t, log_i_t)
 *   C_t = exp(m_{t-1} + log_f_t - m_t) C_{t-1} + exp(log_i_t - m_t) k_t v_t^T   (n_t likewise with k_t)
 *   h_t = q_t^T C_t / (max(|q_t . n_t|, exp(-m_t)) + eps)                         (mlstm.py:214-218)
 * and done_t discards (C, n, m) of the past.  The reference materialises every C_t; here the
 * d x d memory lives in registers and only the carry touches memory.
 *
 *   q, k, v   (B,T,H,d) fp32, d = 32, 64 or 128; k as the cell's element holds it (already divided
 *             by sqrt(d), mlstm.py:196)
 *   log_i, log_f  (B,T,H) fp32: the input-gate pre-activation and -softplus(-f) (mlstm.py:185-186)
 *   c0 (B,H,d,d) indexed [key][value], n0 (B,H,d), m0 (B,H), f0 (B,H): the carry (C, n, m, log_f leaf);
 *             NULL = initialize_carry's zeros / m = -1e9 (mlstm.py:231-240)
 *   h         (B,T,H,d) out: the read-out before the head-wise norm
 *   c_last, n_last, m_last, f_last  next carry, each optional
 * Backward: cotangents dh of h and (dc_last, dn_last, dm_last) of the next carry (NULL = zeros; the
 * log_f leaf has none, no read-out uses it) -> dq, dk, dv, dlog_i, dlog_f and optionally dc0, dn0,
 * dm0.  No per-step state is stored: the kernel walks forward once more, then backward.
 * `workspace`: mxk_mlstm_bwd_workspace_bytes(...) bytes of scratch (six scalars per token and head).
 * ------------------------------------------------------------------------- */
size_t mxk_mlstm_bwd_workspace_bytes(int B, int T, int H, int d);
int mxk_mlstm_f32_fwd(const float* q, const float* k, const float* v, const float* log_i, const float* log_f,
                      const float* c0, const float* n0, const float* m0, const float* f0, const uint8_t* done,
                      float* h, float* c_last, float* n_last, float* m_last, float* f_last, int B, int T, int H, int d,
                      float eps, mxk_stream_t stream);
int mxk_mlstm_f32_bwd(const float* q, const float* k, const float* v, const float* log_i, const float* log_f,
                      const float* c0, const float* n0, const float* m0, const uint8_t* done, const float* dh,
                      const float* dc_last, const float* dn_last, const float* dm_last, float* dq, float* dk, float* dv,
                      float* dlog_i, float* dlog_f, float* dc0, float* dn0, float* dm0, void* workspace,
                      size_t workspace_bytes, int B, int T, int H, int d, float eps, mxk_stream_t stream);

/* ---------------------------------------------------------------------------
 * mLSTM in chunked form on the tensor cores: the same recurrence and reset rule as mxk_mlstm_f32_*
 * (mlstm.py:163-240 under Memoroid.scan_fn) for bf16 q, k, v and a bf16 read-out, gates and carried
 * state in fp32 -- the numerical class of mxk_linattn_bf16_* (bf16 operands, fp32 accumulation), about
 * ten times the throughput of the fp32 kernels.  64-token chunks, one CTA per (batch, head).
 *
 *   q, k, v        (B,T,H,d) bf16, contiguous; k already divided by sqrt(d); d a multiple of 8, at most 64
 *   log_i, log_f   (B,T,H) fp32
 *   c0 (B,H,d,d) fp32 indexed [key][value], n0 (B,H,d), m0 (B,H), f0 (B,H): carried state, NULL = the
 *                  cell's initialize_carry (zeros, m = -1e9)
 *   h              (B,T,H,d) bf16 out;  c_last, n_last, m_last, f_last: next carry, optional
 *   m_steps        optional (B,T,H) fp32 out: the stabiliser after every step, and
 *   chunk_states   optional, mxk_mlstm_bf16_chunk_states_bytes(...) bytes: the bf16 state entering every
 *                  chunk; both are the residuals the backward call needs
 *   status         optional device int, set non-zero if a bounded device-side wait gave up
 * ------------------------------------------------------------------------- */
size_t mxk_mlstm_bf16_chunk_states_bytes(int B, int T, int H, int d);
int mxk_mlstm_bf16_fwd(const void* q, const void* k, const void* v, const float* log_i, const float* log_f,
                       const float* c0, const float* n0, const float* m0, const float* f0, const uint8_t* done,
                       void* h, float* c_last, float* n_last, float* m_last, float* f_last, float* m_steps,
                       void* chunk_states, int* status, int B, int T, int H, int d, float eps, mxk_stream_t stream);

/* Reverse mode of mxk_mlstm_bf16_fwd.  The stabiliser is a gauge of the recurrence: the decay factors are
 * differentiated with it held fixed, and its one real effect on the read-out (eps exp(m_t) in the denominator) and
 * on the stabilised next carry is propagated through m_t = max(m_{t-1} + log_f_t, log_i_t) inside the kernel.
 *   dh             (B,T,H,d) bf16 cotangent of h
 *   c_last, n_last the forward call's next carry (required when dc_last / dn_last is given), m_steps and
 *                  chunk_states its residuals
 *   dc_last (B,H,d,d) [key][value], dn_last (B,H,d), dm_last (B,H): cotangents of the next carry, NULL = zeros
 *   dq, dk, dv     (B,T,H,d) bf16 out;  dlog_i, dlog_f (B,T,H) fp32 out;  dc0, dn0, dm0 optional
 * `done` and the carry's log_f leaf have no cotangent. */
int mxk_mlstm_bf16_bwd(const void* q, const void* k, const void* v, const float* log_i, const float* log_f,
                       const float* c0, const float* n0, const float* m0, const uint8_t* done, const void* dh,
                       const float* c_last, const float* n_last, const float* m_steps, const void* chunk_states,
                       const float* dc_last, const float* dn_last, const float* dm_last, void* dq, void* dk, void* dv,
                       float* dlog_i, float* dlog_f, float* dc0, float* dn0, float* dm0, int* status, int B, int T,
                       int H, int d, float eps, mxk_stream_t stream);

/* ---------------------------------------------------------------------------
 * Gated delta rule (DeltaNet with a scalar forget gate).  The reference has no
 * such cell; this is the new MemoroidCellBase-shaped mixer, defined per head
 * (S is d_v x d_k, a_t = done_t ? 0 : alpha_t) by
 *   S_t = a_t S_{t-1} (I - beta_t k_t k_t^T) + beta_t v_t k_t^T,   o_t = S_t q_t,
 * i.e. Memoroid.scan_fn (memoroid.py:60-91) over the elements
 * (alpha (I - beta k k^T), beta v k^T) with the operator (M_i M_j, U_i M_j + U_j).
 *
 *   q, k, v   (B,T,H,d) bf16, contiguous, d = 128 or 64 (a 64-wide head runs on the
 *             128-wide tiles with their upper half zero-filled by the tensor maps: half the
 *             memory traffic, the arithmetic of d = 128); k is expected L2-normalised
 *   alpha     (B,T,H) fp32 in (0, 1];  beta (B,T,H) fp32
 *   s0        (B,H,d_v,d_k) fp32 carried state, NULL = zeros
 *   o         (B,T,H,d) bf16 out;  s_last (B,H,d_v,d_k) fp32 out, optional
 *   chunk_states  optional residual for the backward call,
 *             mxk_gdelta_chunk_states_bytes(...) bytes (per chunk: the bf16 state
 *             entering it and the solved pseudo-values U)
 *   workspace required scratch of mxk_gdelta_workspace_bytes(...) bytes: a
 *             chunk-parallel preparation kernel leaves every chunk's
 *             (I + diag(beta) L)^-1 diag(beta) there (bf16, 8 KiB per chunk) and the
 *             state-serial kernel reads it back.  Keep it for the backward call on
 *             the same inputs, which reads it too.
 *   status    optional device int, set non-zero if a bounded wait gave up
 * ------------------------------------------------------------------------- */
size_t mxk_gdelta_chunk_states_bytes(int B, int T, int H, int d);
size_t mxk_gdelta_workspace_bytes(int B, int T, int H, int d);
int mxk_gdelta_bf16_fwd(const void* q, const void* k, const void* v, const float* alpha, const float* beta,
                        const float* s0, const uint8_t* done, void* o, float* s_last, void* chunk_states,
                        void* workspace, size_t workspace_bytes, int* status, int B, int T, int H, int d,
                        mxk_stream_t stream);

/* Reverse mode of mxk_gdelta_bf16_fwd.
 *   d_o (B,T,H,d) bf16 cotangent of o;  ds_last (B,H,d,d) fp32 cotangent of the
 *   next carry, NULL = zeros;  chunk_states and workspace as the forward call on the
 *   same inputs left them (both are read only here)
 *   dq, dk, dv (B,T,H,d) bf16 out;  dalpha, dbeta (B,T,H) fp32 out (dalpha is 0
 *   where done, whose steps ignore alpha);  ds0 (B,H,d,d) fp32 out, optional.
 * beta must be non-zero wherever its gradient is wanted (dbeta is written as 0
 * where beta == 0); alpha must lie in (0, 1] (its logarithm is taken). */
int mxk_gdelta_bf16_bwd(const void* q, const void* k, const void* v, const float* alpha, const float* beta,
                        const void* d_o, const void* chunk_states, const void* workspace, const uint8_t* done,
                        const float* ds_last,
                        void* dq, void* dk, void* dv, float* dalpha, float* dbeta, float* ds0, int* status,
                        int B, int T, int H, int d, mxk_stream_t stream);

/* ---------------------------------------------------------------------------
 * Fused Adam step for the training-step harness (the reference trains with
 * optax.adam inside its algorithms, e.g. algorithms/ppo.py:276-279): one flat
 * buffer of n bf16 parameters (n % 8 == 0) with bf16 gradients and fp32
 * moments; bias-corrected update for 1-based `step`; every gradient is
 * multiplied by grad_scale first (1 / world size after a sum all-reduce).
 * ------------------------------------------------------------------------- */
int mxk_adam_bf16(void* params, const void* grads, float* m, float* v, long long n, float lr, float beta1,
                  float beta2, float eps, int step, float grad_scale, mxk_stream_t stream);
/* The same step on fp32 master parameters (optax.adam updates the reference's
 * fp32 params): `master` (n floats) is read, updated and written back, and
 * `params` receives its bf16 rounding in the same pass.  master == NULL is
 * mxk_adam_bf16. */
int mxk_adam_bf16_master(void* params, float* master, const void* grads, float* m, float* v, long long n,
                         float lr, float beta1, float beta2, float eps, int step, float grad_scale,
                         mxk_stream_t stream);

/* ---------------------------------------------------------------------------
 * Row-wise glue of the blocks around a mixer, each fused into one bandwidth-bound pass
 * (bf16 in / out, fp32 arithmetic); used by the training-step harness.
 *
 * LayerNorm (PreNorm, blocks/normalization.py:10-35) and RMSNorm (the norm in front of the
 * cells' output projection, linear_attention.py:114): x, y (rows, D) bf16 with D a multiple of
 * 256 and at most 1024; gamma (and beta for LayerNorm) (D) bf16; mean / rstd (rows) fp32 out
 * (mean unused when rms != 0).  Backward: dx (rows, D) bf16, dgamma / dbeta (D) fp32, reduced over
 * the rows in a fixed order through `workspace` (mxk_norm_bwd_workspace_bytes).
 * Gated residual (blocks/residual.py:53-59): y = x + sigmoid(g) * o over n bf16 elements
 * (n % 8 == 0); backward gives dg and do (dx = dy).
 * Per-head L2 normalisation of q / k for the delta-rule cell: `vectors` head vectors of
 * head_dim (64 or 128) bf16 elements, y = x / max(|x|, eps); with dy != NULL the same call
 * returns dx instead.
 * GELU in its tanh form (flax's nn.gelu default; the FFN block's activation, blocks/ffn.py:16) over n bf16
 * elements (n % 8 == 0): out = gelu(x), or with dy != NULL out = dy * gelu'(x).
 * Column sums of x (rows, cols) bf16 -> out (cols) bf16, added in fp32 in a fixed order through
 * `workspace` (mxk_colsum_workspace_bytes): the bias gradient of a Dense layer (the reference's
 * nn.Dense under autodiff); cols % 8 == 0, else MXK_ERR_UNSUPPORTED.
 * ------------------------------------------------------------------------- */
size_t mxk_norm_bwd_workspace_bytes(long long rows, int D);
int mxk_norm_bf16_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                      long long rows, int D, float eps, int rms, mxk_stream_t stream);
int mxk_norm_bf16_bwd(const void* x, const void* gamma, const float* mean, const float* rstd, const void* dy, void* dx,
                      float* dgamma, float* dbeta, void* workspace, size_t workspace_bytes, long long rows, int D, int rms,
                      mxk_stream_t stream);
int mxk_gated_residual_bf16_fwd(const void* x, const void* g, const void* o, void* y, long long n, mxk_stream_t stream);
int mxk_gated_residual_bf16_bwd(const void* dy, const void* g, const void* o, void* dg, void* d_o, long long n,
                                mxk_stream_t stream);
int mxk_l2norm_heads_bf16(const void* x, const void* dy, void* out, long long vectors, int head_dim, float eps,
                          mxk_stream_t stream);
int mxk_gelu_bf16(const void* x, const void* dy, void* out, long long n, mxk_stream_t stream);
size_t mxk_colsum_workspace_bytes(long long rows, int cols);
int mxk_colsum_bf16(const void* x, void* out, void* workspace, size_t workspace_bytes, long long rows, int cols,
                    mxk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MXK_H_ */
