/* libstu_b200.so -- C ABI of the B200 (sm_100a) kernels for the Flash STU token loop.
 *
 * The reference (hazan-lab/flash-stu-2) is pure PyTorch and has no FFI layer; its operator boundary is
 * the set of Python modules cited beside each entry point below (paths inside the reference
 * repository).  A host binding calls these functions with DEVICE pointers (e.g. tensor.data_ptr()),
 * plain sizes/strides in ELEMENTS, and the CUDA stream to launch on.
 *
 * Conventions
 *   dtype      0 = float32, 1 = bfloat16 (storage and rounding points; accumulation is fp32)
 *   stream     a cudaStream_t passed as void*
 *   return     0 = ok; <0 = argument error detected on the host before any launch
 *              (-1 dtype, -2 shape, -3 alignment, -4 unsupported configuration, -5 null pointer,
 *              -7 built-in scratch too small);
 *              >0 = cudaError_t from the launch.  Nothing throws, aborts or traps.
 *   ownership  the caller allocates every input, output, cache and scratch buffer; the library keeps no
 *              pointer after a call returns (except the status word registered below) and never
 *              allocates or synchronises.
 *   status     device-side problems (bounded waits that expired, ids/positions out of range) are written
 *              to the int registered with stu_set_status_word(); 0 means none.
 *   pos        int32 [B][2] device array: pos[2*b] = tokens of sequence b already cached,
 *              pos[1] = arrival counter (must be 0 between calls).  Kernels that append to a cache
 *              advance it themselves, so a captured CUDA graph can be replayed without new arguments.
 *   history    projected STU inputs, [B][d][2][Lh]: element (b, c, t) at ((b*d + c)*2 + (t&1))*Lh + (t>>1)
 */
#ifndef STU_B200_H
#define STU_B200_H

#ifdef __cplusplus
extern "C" {
#endif

int stu_b200_version(void);

/* Registers, for the CURRENT device, the device int that kernels launched on that device set on a device-side
 * problem (NULL to unregister).  One word per device: a process that drives several GPUs registers one word on
 * each, with that GPU current. */
int stu_set_status_word(int* device_status);

/* Failure-detection test hook (no counterpart in the reference): arms ONE injected fault for the next tcgen05 GEMM
 * launched by stu_linear -- the copies of its first pipeline stage are never issued -- and shortens every bounded
 * device-side wait to wait_ms milliseconds.  That launch must report status 3 and return; the GPU context stays
 * usable.  wait_ms = 0 disarms and restores the two-second bound. */
int stu_test_inject_wait_expiry(int wait_ms);

/* y[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) * w.
 * Replaces torch.nn.RMSNorm / LigerRMSNorm as used in flash_stu/layers/stu_layer.py:32-36,67-71,
 * flash_stu/layers/attention_layer.py:33-43 and flash_stu/model.py:90-96,173. */
int stu_rmsnorm(const void* x, const void* w, void* y, int rows, int d, long long x_row_stride,
                long long y_row_stride, float eps, int dtype, void* stream);

/* y[r, c] = act(y[r, c] + bias[c]) in place (bias may be NULL); act: 0 none, 1 ReLU, 2 GELU (erf form), 3 tanh,
 * 4 SiLU.  The nn.Linear bias + activation modules of the MiniSTU post-MLP (mini_stu/stu.py:171-211) and the SiLU
 * between the projections of the STU sandwich (flash_stu/layers/stu_layer.py:52,84). */
int stu_bias_act(void* y, const void* bias, long long rows, int cols, long long y_row_stride, int act, int dtype,
                 void* stream);

/* out[r,:] = table[ids[r],:] (int64 ids).  Replaces nn.Embedding at flash_stu/model.py:152. */
int stu_embed(const long long* ids, const void* table, void* out, int rows, int d, int vocab, int* status,
              int dtype, void* stream);

/* y = epilogue(x[M,K] @ W[N,K]^T); element (n,k) of W at W[n*w_row_stride + k*w_k_stride].
 *   epilogue 0  y = acc                       nn.Linear: attention.py:74,101; model.py:176; `x @ M_inputs` stu.py:87
 *            1  y = resid + round(acc)        the x.add_(...) of stu_layer.py:93,96 / attention_layer.py:56,62
 *            2  y = round(gelu_tanh(round(x@W^T))) * round(x@W2^T)     swiglu.py:22-28
 *            3  scatter round(acc) into the history `y` (N channels, hist_T tokens per sequence starting at
 *               time hist_t0, hist_Lh elements per parity row): the projected input `x @ M_inputs`
 *            5  y[m*y_row_stride + (n / hist_T)*resid_row_stride + (n % hist_T)] = acc: the output columns come in
 *               blocks of hist_T, consecutive blocks resid_row_stride elements apart (resid itself is not read).  Used
 *               for the distilled-LDS features h@C of mini_stu/stu_lds.py:337, written straight into the
 *               [tokens, F*d] operand of the contraction with M (stu_lds.py:389-393)
 *   norm_w     when non-NULL, x is RMS-normalised with this weight (eps) inside the kernel; only fused for
 *              decode shapes (see stu_linear_can_fuse_norm), otherwise -4.
 *   backend    0 auto (M<=64: the token-step kernels - bf16 with 9..64 rows: tcgen05 with the weights as the 128-row
 *              operand and K split over a thread-block cluster; up to 8 rows, fp32 or a fused norm: weight-streaming
 *              mma.sync/FMA kernels; larger M, bf16 aligned: tcgen05+TMA GEMM; else CUDA-core GEMM),
 *              1 CUDA-core, 2 tcgen05 GEMM, 3 token-step kernels. */
/* epilogue flags: 0x100 = W is lower triangular (k-blocks above the diagonal are skipped); 0x200 = launch with
 * programmatic stream serialization: the kernel fetches W (which the preceding kernel must not write) while that
 * kernel drains, and reads x only after it has completed (skinny shapes, M <= 64; ignored otherwise);
 * 0x400 = let the next 0x200 launch start at once. */
int stu_linear(const void* x, long long x_row_stride, const void* W, long long w_row_stride, long long w_k_stride,
               const void* W2, const void* resid, long long resid_row_stride, void* y, long long y_row_stride,
               int M, int N, int K, int epilogue, int hist_T, int hist_t0, int hist_Lh, const void* norm_w,
               float eps, int dtype, int backend, void* stream);
int stu_linear_can_fuse_norm(int M, int N, int K, int epilogue, int dtype);

/* taps[c][j] = fp[2j][c] for fp = phi @ M_filters ([L,d], model dtype): the even taps that survive when the
 * plus and minus branches of flash_stu/utils/stu_utils.py:223-227 are added (flash_stu/modules/stu.py:88,120). */
int stu_taps_even(const void* fp, void* taps, int L, int d, int Lh, int dtype, void* stream);

/* Prefill convolution of the approx STU variant: for t in [t0, t_end)
 *   x[b, t-t0, c] += round(2 * sum_{j even, j<=t} fp[j,c] * hist(b,c,t-j))
 * i.e. spectral_plus + spectral_minus of flash_stu/modules/stu.py:95-98,120 (torch.fft path
 * flash_stu/utils/stu_utils.py:208-228), added to the residual stream.  hist must already hold the
 * projected inputs of times [0, t_end).  yT is scratch with the history layout and y_Lh elements per
 * parity row (y_Lh >= ceil(t_end/2)); yT must be 16-byte aligned and y_Lh a multiple of 8 (bf16) or 4 (fp32),
 * because the residual add reads it in 16-byte vectors: anything else returns -3 before a kernel is launched.
 * use_tensor_cores=1 (bf16 only) runs the Toeplitz product on tensor cores, 0 the fp32 CUDA-core kernel. */
int stu_conv_prefill_approx(const void* hist, const void* taps, void* yT, void* x, long long x_bstride,
                            long long x_tstride, int B, int d, int Lh, int y_Lh, int t0, int t_end, int dtype,
                            int use_tensor_cores, void* stream);

/* The same prefill convolution for callers that cannot allocate device memory (a server whose own arena
 * already owns all of HBM, or a steady-state loop under a no-allocation rule): the scratch is a fixed
 * 32 MiB array inside the library image instead of the caller's yT.  This entry point has no counterpart
 * in the reference.  Returns -7 when B*d*2*roundup8(ceil(t_end/2)) elements exceed 32 MiB.  The first
 * call on a device resolves the array's address (make it outside stream capture); all calls on a device
 * share the array, which keeps the previous call's contents and needs no clearing; calls overlapping on
 * one GPU race.  Never calls cudaMalloc/cudaFree. */
int stu_conv_prefill_approx_static(const void* hist, const void* taps, void* x, long long x_bstride,
                                   long long x_tstride, int B, int d, int Lh, int t0, int t_end, int dtype,
                                   int use_tensor_cores, void* stream);

/* The same prefill convolution (bf16) on the tcgen05 tensor cores: per channel the Toeplitz product is regrouped by
 * block distance so that one instruction covers every 128-position output block at once (N up to 512), the
 * accumulator of 4096 positions x 16 parity rows lives in tensor memory, the history chunks and the Toeplitz blocks
 * arrive by cp.async.bulk.tensor, the latter straight from the reversed tap table taps8 of stu_taps_rev8 through a
 * tensor map with an overlapping row stride.  Replaces the same reference lines as stu_conv_prefill_approx
 * (flash_stu/modules/stu.py:95-98,120; flash_stu/utils/stu_utils.py:208-228).  Needs Lh % 128 == 0 (-4 otherwise:
 * use stu_conv_prefill_approx), hist, taps8 and yT 16-byte aligned, y_Lh % 8 == 0 (-3).  status receives 9 when a
 * bounded pipeline wait ran out. */
int stu_conv_prefill_approx_tc5(const void* hist, const void* taps8, void* yT, void* x, long long x_bstride,
                                long long x_tstride, int B, int d, int Lh, int y_Lh, int t0, int t_end, int* status,
                                int dtype, void* stream);

/* The token-step kernels (RMSNorm, the decode linears, the attention and STU decode kernels) are launched with the
 * programmatic-stream-serialization attribute: each fetches its weights while the kernel before it drains and waits
 * (griddepcontrol.wait) before it touches anything that kernel writes.  stu_set_programmatic_launch(0) turns the
 * launches that follow back into plain stream-ordered ones (as STU_B200_DISABLE_PDL=1 does from the start) and
 * returns the previous setting; a captured CUDA graph keeps what it was captured with.  No counterpart in the
 * reference. */
int stu_set_programmatic_launch(int on);

/* Profiling aid of stu_conv_prefill_approx_tc5: while a device buffer of 128 64-bit words is registered, CTA 0 of
 * every launch writes nanosecond stamps of its first 8 units into it (16 words per unit: 0 accumulator free,
 * 1 first operands ready, 2 last MMA issued, 3 accumulator complete, 4 epilogue done; per phase: 5 stage free,
 * 6 history chunk landed, 7 stage ready).  NULL switches it off.  No counterpart in the reference. */
int stu_conv_prefill_set_timeline(void* device_words);

/* One cached decode step of an approx STU layer, fused:
 *   out[b,:] = x[b,:] + STU(rmsnorm(x[b,:]) * norm_w)   at time t = pos[2*b]; appends to hist, advances pos.
 * MinT is M_inputs transposed ([d_out][d_in]).  The reference has no such step (its STU layers keep no
 * cache, flash_stu/layers/stu_layer.py:99-119); the result equals row t of the full-prefix forward of
 * flash_stu/layers/stu_layer.py:78-93.  out must not alias x.
 * taps8 (bf16 only, may be NULL) is the table made by stu_taps_rev8; with it the step runs on mma.sync tensor
 * cores, without it on CUDA cores (one warp per sequence and channel).
 * Flags OR-ed into dtype: 0x800 = every sequence stands at the same position (checked on the device, status 6
 * if not): selects the kernel that owns 8 channels x 8 sequences per CTA and shares the taps between sequences;
 * 0x400 = let a following stu_linear launched with 0x200 start before this kernel has finished.
 */
int stu_decode_approx(const void* x, long long x_row_stride, const void* norm_w, const void* MinT, void* hist,
                      const void* taps, const void* taps8, int* pos, void* out, long long out_row_stride, int B,
                      int d, int Lh, float eps, int* status, int dtype, void* stream);

/* taps8[e][c][u] = taps[c][Lh-1-(u+e)] (0 past the end), e = 0..7, row pitch Lh+8: the even-tap table reversed
 * and stored in all eight 16-byte alignments, so that the decode kernel's tap operand is an aligned
 * 16-byte load at every position.  bf16, Lh % 8 == 0.  Derived data, no counterpart in the reference. */
int stu_taps_rev8(const void* taps, void* taps8, int d, int Lh, int dtype, void* stream);

/* Channel shard of stu_decode_approx for tensor parallelism (the reference is single-GPU; the STU sub-layer is
 * flash_stu/layers/stu_layer.py:78-93): x [B, d_in] is the full layer input, MinT [d_ch][d_in], hist
 * [B][d_ch][2][Lh], taps8 [8][d_ch][Lh+8] and out [B, d_ch] hold the d_ch channels owned by the caller.  With
 * add_residual = 0 out receives the STU output alone (to be all-gathered and added to the residual stream);
 * add_residual = 1 needs d_in == d_ch.  bf16 only, all sequences at one position (status 6 otherwise),
 * d_in, d_ch, Lh multiples of 8.  dtype takes the launch flags 0x200 / 0x400 of stu_decode_approx. */
int stu_decode_approx_shard(const void* x, long long x_row_stride, const void* norm_w, const void* MinT, void* hist,
                            const void* taps8, int* pos, void* out, long long out_row_stride, int B, int d_in,
                            int d_ch, int Lh, float eps, int add_residual, int* status, int dtype, void* stream);

/* The same fused decode step (whole layer: d_in == d_ch, add_residual = 1; or a channel shard) as a persistent
 * bulk-copy pipeline: one CTA per SM owns rows of 8 sequences x 8 channels; the history and taps of 256 positions
 * per cp.async.bulk.tensor copy pair go through a 4-stage shared-memory ring, the dot products run on tensor cores,
 * and a separate warp group projects the new token under the stream.  A row is summed inside one CTA, slices in
 * order, so results do not depend on the SM count.  Replaces the same reference lines as stu_decode_approx
 * (flash_stu/modules/stu.py:85-98,120 for one new position).  bf16, all sequences at one position (status 6
 * otherwise), d_in, d_ch, Lh multiples of 8; status 7 = a bounded pipeline wait ran out.  dtype takes the launch
 * flags 0x200 (start while the preceding kernel of the stream is still running: only the projection waits for it)
 * and 0x400. */
int stu_decode_approx_pipelined(const void* x, long long x_row_stride, const void* norm_w, const void* MinT,
                                void* hist, const void* taps8, int* pos, void* out, long long out_row_stride, int B,
                                int d_in, int d_ch, int Lh, float eps, int add_residual, int* status, int dtype,
                                void* stream);

/* One cached token step of a whole approx STU layer -- x += STU(norm(x)); x += MLP(norm(x)), the decode form of
 * flash_stu/layers/stu_layer.py:78-97 with flash_stu/modules/stu.py:85-98,120 and flash_stu/modules/swiglu.py:22-29 --
 * as ONE persistent cooperative kernel for up to 8 sequences at one common position (bf16).  The kernel pipelines
 * across launches: while its projection / MLP warps finish position t, its streaming warps already compute the
 * history partial sums of position t+1 (they need nothing step t produces) and leave them in `workspace` for the next
 * launch.  mode 0: the token step (needs the partial sums of the current position in the workspace: status 8
 * otherwise; advances pos).  mode 1: only compute the partial sums of the current position (first step after a
 * prefill).  workspace: stu_block_step_workspace_bytes(d, I) bytes, 256-byte aligned, zeroed once by the caller (an
 * all-zero workspace is the correct state for position 0), private to one layer's cache.  out may alias x.
 * MinT [d][d] rows = output channels; Wg, Wu [I][d]; Wd [d][I].  d, I, Lh multiples of 8, B <= 8. */
long long stu_block_step_workspace_bytes(int d, int I);
int stu_block_decode_step(const void* x, long long x_row_stride, const void* stu_norm_w, const void* MinT, void* hist,
                          const void* taps8, int* pos, const void* mlp_norm_w, const void* Wg, const void* Wu,
                          const void* Wd, void* out, long long out_row_stride, int B, int d, int I, int Lh,
                          float eps_stu, float eps_mlp, void* workspace, long long workspace_bytes, int mode,
                          int* status, int dtype, void* stream);

/* ---- full STU variant (flash_stu/modules/stu.py:100-118, mini_stu/stu.py:240-269): U+-[b,t,k,i] =
 * sum_j (+-1)^j phi[j,k] x[b,t-j,i] contracted with M_phi_plus / M_phi_minus.  The filters are shared by all
 * channels, so per filter the convolution is three GEMMs (stu_linear with epilogue | 0x100 = lower-triangular
 * weight) of history rows with Toeplitz matrices, combined into the token-major operand of the contraction. */

/* x [B, t_end-t0, d] (token-major) -> history layout, times [t0, t_end). */
int stu_to_history(const void* x, long long x_bstride, long long x_tstride, void* hist, int B, int d, int Lh, int t0,
                   int t_end, int dtype, void* stream);

/* out[kind][m][s], kind 0..2, S x S each with row pitch ld, from one filter column f[j*f_stride], j < L:
 * kind 0: f[2(m-s)] (even taps); kind 1: f[2(m-s)+1] (odd taps feeding parity-1 outputs from parity-0 inputs);
 * kind 2: f[2(m-s)-1] (odd taps feeding parity-0 outputs from parity-1 inputs); zero above the diagonal. */
int stu_toeplitz(const void* f, long long f_stride, int L, void* out, int S, long long ld, int dtype, void* stream);

/* U[(b,t-t0)][k*d+i] = E+Q and, with both_signs, U[..][(K+k)*d+i] = E-Q, for E,Q [B*d*2][ldE] in history row
 * order (the even-tap and odd-tap products of filter k). */
int stu_full_combine(const void* E, const void* Q, long long ldE, void* U, long long ldU, int B, int d, int K, int k,
                     int both_signs, int t0, int t_end, int dtype, void* stream);

/* One cached decode step of the full variant, around one GEMM G = hist_rows @ PhiT^T (stu_linear, M = B*d*2,
 * N = 2K, K = Lh): prepare appends x_t at time pos[0] and rebuilds PhiT [2K][Lh] (time-reversed even / odd
 * taps for that position); combine forms U+- [B][2*K*d] from G and (advance != 0) moves every position on.
 * The reference has no cached STU step (flash_stu/layers/stu_layer.py:99-119). */
int stu_full_decode_prepare(const void* x, long long x_row_stride, void* hist, const void* phi, const int* pos,
                            void* PhiT, int B, int d, int K, int L, int Lh, int* status, int dtype, void* stream);
int stu_full_decode_combine(const void* G, long long ldG, int* pos, void* U, int B, int d, int K, int both_signs,
                            int Lh, int advance, int dtype, void* stream);

/* ---- distilled-LDS variant (mini_stu/stu_lds.py:213-394): per channel h_t = A*h_{t-1} + B*x_t (D modes, float64),
 * U[f] = sum_n h[n] C[n,f], y = sum_{f,i} U[f,i] M[f,i,o].  Prefill outputs go through the full-variant entry
 * points above with the impulse responses G[j,f] = sum_n C[n,f] B[n] A[n]^j as filters. */

/* h [B*d][D] (float64) <- state after the Tn inputs held in hist; replaces the scan of mini_stu/stu_lds.py:17-99 for
 * the purpose of seeding the decode. */
int stu_lds_final_state(const void* hist, double* h, const double* A, const double* Bv, int B, int d, int Lh, int Tn,
                        int D, int dtype, void* stream);

/* Chunked-scan prefill of the distilled LDS (mini_stu/stu_lds.py:17-99 lds_scan_kernel / run_lds_scan, :181-200
 * affine_scan_with_fixed_a, :280-338 FixedDiagonalLDS.forward): runs h = A*h + B*x[b,t,i] in float64 over the Tn
 * positions of every (sequence, channel) of x [B,Tn,d]; at the start of every chunk of Ck positions writes the carried
 * state, rotated into a balanced basis (z = Vs^T h, Vs [D][R] float64), and the chunk's inputs into
 * Z [B][ceil(Tn/Ck)][d][KZ] (bf16: z_hi | z_lo | z_hi | x, KZ = 3R+Ck; fp32: z | x, KZ = R+Ck), and the final state into
 * hfin [B*d][D] (bit-identical to stu_lds_final_state).  The features of all chunks of a sequence are then ONE
 * stu_linear call with epilogue 5 on Z (see flash_stu_2_b200/mini_stu.py for the constant operand).  R % 8 == 0,
 * Ck % 8 == 0, D <= 256.  dtype | 0x1000: the caller has checked that every Bv[n] is exactly 1 (faster kernel, same
 * bits). */
int stu_lds_chunk_scan(const void* x, long long x_bstride, long long x_tstride, const double* A, const double* Bv,
                       const double* Vs, void* Z, double* hfin, int B, int d, int Tn, int D, int R, int Ck, int dtype,
                       void* stream);

/* One recurrent step (mini_stu/lds.py:95-101): h updated in place, U [B][F*d] = features in the row order of M. */
int stu_lds_decode_features(const void* x, long long x_row_stride, double* h, const double* A, const double* Bv,
                            const void* C, void* U, int B, int d, int D, int F, int dtype, void* stream);

/* Sliding-window attention for the Tn new tokens in qkv [B,Tn,3*H*hd] (c_attn output) against a ring
 * cache of W >= window+1 slots ([B][W][H*hd] each; token t in slot t % W), ALiBi slopes [H] (fp32) and tanh
 * soft-capping; out [B,Tn,H*hd] (heads merged, before c_proj).  update_cache=1 stores the new keys/values
 * and advances pos by Tn.  Replaces flash_attn_func as called at flash_stu/modules/attention.py:90-99 and
 * the torch.cat cache of attention.py:82-88. */
int stu_swa_forward(const void* qkv, void* k_ring, void* v_ring, int* pos, const float* slopes, void* out, int B,
                    int Tn, int H, int hd, int W, int window, float softcap, int update_cache, int dtype,
                    void* stream);

/* Next token from last-position logits [B,V]: temperature, clamp(+-1e4), top-k, top-p, then argmax or an
 * inverse-CDF draw from uniforms[b]; writes int64 ids to out[b*out_stride].  Replaces
 * flash_stu/model.py:268-299 (torch.multinomial is replaced by the reproducible draw).
 * top_k <= 0 and top_p outside (0,1) disable the filters; top_p needs top_k (<= 1024). */
int stu_sample(const void* logits, long long ld, int B, int V, float temperature, int top_k, float top_p,
               int do_sample, const float* uniforms, long long* out, long long out_stride, int* status, int dtype,
               void* stream);

/* The same decode step for a caller that computed the projected input of the new token itself as one GEMM over the
 * whole batch: xp [B, d_ch] = (rmsnorm(x) * norm_w) @ M_inputs (flash_stu/modules/stu.py:87), bf16.  Appends xp to
 * hist, advances pos, out = (add_residual ? x : 0) + round(2 * taps . hist).  For batches of more than 8 sequences,
 * where the per-row projection inside stu_decode_approx_pipelined costs more than the row's stream.  x may be NULL
 * when add_residual = 0. */
int stu_decode_approx_projected(const void* x, long long x_row_stride, const void* xp, long long xp_row_stride,
                                void* hist, const void* taps8, int* pos, void* out, long long out_row_stride, int B,
                                int d_ch, int Lh, int add_residual, int* status, int dtype, void* stream);

/* Attention of a prefill that starts at position 0 (every pos[2b] == 0, checked on the device: status 11 otherwise)
 * on the tcgen05 tensor cores: bf16, head dimension 128.  Same semantics and outputs as stu_swa_forward for that
 * case (flash_stu/modules/attention.py:72-101): 128 queries x one head per CTA, S = Q K^T and O += P V as
 * tcgen05.mma with S, O in tensor memory, Q / K tiles / V^T tiles by cp.async.bulk.tensor, softmax by four warps
 * against a lazily moved row maximum; update_cache stores the last W tokens in the rings and advances pos by Tn.
 * vt_scratch: stu_swa_prefill_scratch_elems(B, Tn, H, 128) bf16 elements, 16-byte aligned (V transposed per head by
 * a kernel of its own).  -4 for other head dimensions. */
long long stu_swa_prefill_scratch_elems(int B, int Tn, int H, int hd);
int stu_swa_prefill_tc5(const void* qkv, void* vt_scratch, void* k_ring, void* v_ring, int* pos, const float* slopes,
                        void* out, int B, int Tn, int H, int hd, int W, int window, float softcap, int update_cache,
                        int* status, int dtype, void* stream);

/* ---- exchange between the GPUs of a tensor-parallel group, fused into the token loop's kernels ----------------
 * The reference is single-GPU (its sub-layers: flash_stu/layers/stu_layer.py:78-98,
 * flash_stu/layers/attention_layer.py); these calls replace the all-gather after a channel-sharded STU sub-layer and the
 * all-reduce after a column-sharded MLP / attention sub-layer for the one new token of a cached decode step.  Every
 * rank owns one peer buffer (stu_peer_alloc) that the other ranks map (stu_peer_export / stu_peer_open, CUDA IPC); it
 * holds, per exchange point of the token step, an inbox, one arrival counter per sender, a send counter and a CTA
 * counter.  A producing kernel stores its rows straight into every rank's inbox (plain stores to peer memory) and its
 * last CTA raises the sender's counter on every rank; stu_peer_combine waits (bounded) for all senders.  No load ever
 * targets another GPU's memory.
 *
 * An exchange descriptor (stu_peer_dest_bytes() bytes of the sender's device memory) is laid out as
 *   int n, pad;  void* dest[8];  unsigned* flag[8];  unsigned* epoch;  unsigned* ctr;
 * dest[p] = where this rank's rows start inside rank p's inbox, flag[p] = rank p's arrival counter for this sender,
 * epoch / ctr = this rank's send counter and CTA counter of the exchange (both start at 0). */
int stu_peer_dest_bytes(void);
int stu_peer_alloc(void** ptr, long long bytes);            /* zero-filled; a dedicated cudaMalloc allocation */
int stu_peer_free(void* ptr);
int stu_peer_export(void* ptr, void* handle64);             /* 64-byte inter-process handle of the allocation */
int stu_peer_open(const void* handle64, void** ptr);        /* map another rank's allocation */
int stu_peer_close(void* ptr);
int stu_peer_write(void* dst, const void* host_src, long long bytes);   /* synchronous host -> buffer copy */
int stu_peer_read(void* host_dst, const void* src, long long bytes);    /* synchronous buffer -> host copy */

/* y = x[M,K] @ W[N,K]^T (bf16, M <= 64: the weight-streaming kernel) stored into every rank's inbox through the
 * exchange descriptor, rows dest_row_stride elements apart; -4 for shapes that kernel does not take. */
int stu_linear_push(const void* x, long long x_row_stride, const void* W, long long w_row_stride, int M, int N, int K,
                    const void* peer_dest, long long dest_row_stride, int dtype, void* stream);

/* stu_decode_approx_pipelined for a channel shard (add_residual = 0) whose d_ch outputs per sequence go into every
 * rank's inbox through the exchange descriptor instead of `out`. */
int stu_decode_approx_push(const void* x, long long x_row_stride, const void* norm_w, const void* MinT, void* hist,
                           const void* taps8, int* pos, const void* peer_dest, long long dest_row_stride, int B,
                           int d_in, int d_ch, int Lh, float eps, int* status, int dtype, void* stream);

/* Receiving side of one exchange, one CTA per row: waits until all n_ranks arrival counters (flags) have reached
 * this rank's send counter (epoch), then x[row] = round(x[row] + round(sum of the `slots` inbox blocks' rows)) and,
 * with norm_w, xn[row] = RMSNorm(x[row]) * norm_w (the next sub-layer's normalisation).  inbox blocks are slot_stride
 * elements apart, their rows in_row_stride.  The wait gives up after wait_ms (0: two seconds): status 10, x untouched.
 * bf16, d % 8 == 0, d <= 16384. */
int stu_peer_combine(void* x, long long x_row_stride, const void* inbox, long long slot_stride, long long in_row_stride,
                     int slots, const void* flags, int n_ranks, const void* epoch, const void* norm_w, void* xn,
                     long long xn_row_stride, float eps, int rows, int d, int* status, int wait_ms, int dtype,
                     void* stream);

/* One exchange of the token step in ONE launch, one CTA per row: the CTA copies this rank's contribution of its row
 * (src [rows, cols]; gather != 0: the rank's cols = d / n channels, gather == 0: a full-width partial sum) into every
 * rank's inbox with 16-byte stores, raises this sender's counter of the row on every rank, waits (bounded, wait_ms,
 * 0: two seconds; status 10) for the other senders of the row, then x[row] = round(x[row] + round(sum)) and, with
 * norm_w, xn[row] = RMSNorm(x[row]) * norm_w.  xchg = the exchange's record in this rank's device memory
 * (stu_peer_xchg_bytes() bytes):
 *   int n, rank;  void* inbox[8];  unsigned* flag[8];  unsigned* epoch;
 * inbox[p] = rank p's inbox of the exchange ([slots][rows][d], blocks slot_stride elements apart), flag[p] = rank p's
 * counters of the exchange ([n senders][rows]), epoch = this rank's [rows] exchange counts (all start at 0). */
int stu_peer_xchg_bytes(void);
int stu_peer_exchange(const void* xchg, void* x, long long x_row_stride, const void* src, long long src_row_stride,
                      int cols, int gather, long long slot_stride, const void* norm_w, void* xn,
                      long long xn_row_stride, float eps, int rows, int d, int* status, int wait_ms, int dtype,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* STU_B200_H */
