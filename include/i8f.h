/*
 * libi8f -- C ABI of the B200 (sm_100a) W8A8 linear hot path.
 *
 * Each entry point replaces one piece of the Python/Triton hot path of the
 * ComfyUI-INT8-Fast node pack; the file:line next to it names what it stands
 * in for (paths are relative to that project).
 *
 * Conventions
 *   - Every function returns I8F_OK (0) or a negative I8F_ERR_* code and never
 *     throws; i8f_last_error() returns a thread-local description of the
 *     last failure.
 *   - All data pointers are device pointers on the current CUDA device and are
 *     only borrowed until the enqueued work finishes.  Nothing is allocated,
 *     nothing synchronises: work is enqueued on `stream` (a cudaStream_t
 *     passed as void*; NULL means the legacy default stream).
 *   - Matrices are row-major; `ld*` are row pitches in ELEMENTS.
 *   - dtype codes: I8F_BF16, I8F_F16, I8F_F32.
 *   - Kernels that feed the tensor cores through TMA need 16-byte aligned
 *     base pointers and row pitches that are multiples of 16 bytes; this is
 *     checked and reported as I8F_ERR_ALIGNMENT, never left undefined.
 *   - Device-side waits are bounded; a wait that runs out is recorded in a
 *     device status word readable with i8f_device_status().
 */
#ifndef I8F_H_
#define I8F_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define I8F_VERSION 100

#define I8F_OK 0
#define I8F_ERR_INVALID_ARG (-1)
#define I8F_ERR_ALIGNMENT (-2)
#define I8F_ERR_UNSUPPORTED (-3)
#define I8F_ERR_CUDA (-4)
#define I8F_ERR_DEVICE (-5)
#define I8F_ERR_WORKSPACE (-6)

#define I8F_BF16 0
#define I8F_F16 1
#define I8F_F32 2

/* weight-scale granularity */
#define I8F_WSCALE_TENSOR 0  /* one fp32 value in device memory */
#define I8F_WSCALE_CHANNEL 1 /* fp32[N] in device memory */

/* epilogue rounding order */
#define I8F_EPI_PYTORCH 0 /* round after scaling, round again after the bias add */
#define I8F_EPI_SINGLE 1  /* one rounding after scale and bias */

/* Library version (I8F_VERSION of the build). */
int i8f_version(void);

/* Number of kernels this library has launched in the process so far (all devices, all streams); a host-side
 * counter for accounting, e.g. launches per step = the difference around a step.  No counterpart in the reference. */
uint64_t i8f_launch_count(void);

/* Thread-local text of the last error returned on this thread ("" if none). */
const char* i8f_last_error(void);

/* I8F_OK if the current device is compute capability 10.0, else I8F_ERR_DEVICE.
 * Replaces the `x.is_cuda` / Triton-availability dispatch at int8_quant.py:72, :103
 * with a hard requirement. */
int i8f_device_check(void);

/* Reads (and if `reset` is non-zero clears) the device status word of the
 * current device.  0 means no bounded wait has run out since the last reset.
 * Synchronises the device; meant for tests and diagnostics. */
int i8f_device_status(int* status_out, int reset);

/* Diagnostic, host only (no device needed): the tile configuration the GEMM entry points choose for an
 * [M,K] x [N,K]^T problem with 1-byte (int8) or 2-byte (bf16 / fp16) operands on a GPU with `sm_count_or_0` SMs
 * (0: the current device, 148 if there is none), ignoring the environment switches: tile_rows x tile_cols,
 * ctas_per_tile (2 for the 256 x 256 tile of a CTA pair; doubled again when two CTAs of a cluster split the tile's K
 * range) and k_split (1 or 2).  No counterpart in the reference, whose Triton kernels leave this to the autotuner
 * (int8_fused_kernel.py:81-89). */
int i8f_gemm_plan(int64_t M, int64_t N, int64_t K, int elem_bytes, int sm_count_or_0, int* tile_rows, int* tile_cols,
                  int* ctas_per_tile, int* k_split);

/* Diagnostic: launches one CTA that waits on a barrier nothing signals.  The device-side wait gives up after
 * `limit_cycles` SM clocks, the kernel ends normally and i8f_device_status() then reads 199.  This is how the
 * time-out path of every in-kernel wait is exercised without hanging or faulting the GPU.  No counterpart in
 * the reference. */
int i8f_selftest_bounded_wait(int64_t limit_cycles, void* stream);

/* Per-token absmax quantisation, optionally fused with the 128-block
 * Walsh-Hadamard rotation.
 *   x [M,K] (x_dtype) -> q int8 [M,K], scale fp32 [M]
 *   scale = max(absmax/127, 1e-30); q = clamp(rint(x * (1/scale)), -128, 127)
 * hadamard128 != 0 first rotates every 128-block of a row (K % 128 == 0
 * required) and rounds the result to x_dtype; x_rot_out (may be NULL) receives
 * that rotated tensor in x_dtype with pitch ldx.
 * Replaces triton_quantize_rowwise (int8_fused_kernel.py:10-73),
 * quantize_int8_axiswise (int8_quant.py:28-31) and rotate_activation
 * (quarot.py:73-102) as called from int8_quant.py:741-744. */
int i8f_quant_rowwise(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                      int8_t* q, int64_t ldq, float* scale, int hadamard128,
                      void* x_rot_out, void* stream);

/* The activation quantiser with the element-wise step in front of a quantised linear folded in.  The three entry
 * points below have no counterpart in the reference, which leaves these steps to the model's own PyTorch code
 * (a diffusion transformer runs LayerNorm -> modulate -> Linear, GELU -> Linear and a per-head RMS norm of q and k
 * around every quantised linear, each a full pass over the activations that the quantiser then reads again).
 * Their arithmetic is specified completely, every rounding and the order of every sum, in
 * comfyui-int8-fast_b200/csrc/quant_prologue.cu; rows are at most 16384 elements, dtype I8F_BF16 or I8F_F16.
 *
 * y = rnd(rnd((x - mean) * rstd) * rnd(1 + scale[k]) + shift[k]) over each row of x [M,K] (LayerNorm without
 * affine parameters, eps added to the variance; shift, scale: [K] in x_dtype), then q, row_scale as
 * i8f_quant_rowwise computes them from y.  y_out (may be NULL) receives y in x_dtype with pitch ldy. */
int i8f_quant_rowwise_ln_modulate(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                                  const void* shift, const void* scale, float eps,
                                  int8_t* q, int64_t ldq, float* row_scale, void* y_out, int64_t ldy, void* stream);

/* y = [ x_plain [M,K0] | rnd(GELU_tanh(x_gelu [M,K1])) ] row by row (either part may be empty), then q [M,K0+K1],
 * row_scale as i8f_quant_rowwise computes them from y.  The GELU is x * sigmoid(2u), u = sqrt(2/pi) (x + 0.044715
 * x^3), evaluated in correctly rounded fp32 operations only.  y_out (may be NULL) receives y.  Large inputs read
 * rnd(GELU(x)) from a table of all 65536 16-bit values (same bits): 256 KB inside the library image, filled by a
 * kernel on this call's stream the first time a device needs it; calls on other streams are ordered behind that
 * build with an event, nothing is allocated and the host never waits. */
int i8f_quant_rowwise_gelu(const void* x_plain, int64_t K0, int64_t ld0, const void* x_gelu, int64_t K1, int64_t ld1,
                           int x_dtype, int64_t M, int8_t* q, int64_t ldq, float* row_scale,
                           void* y_out, int64_t ldy, void* stream);

/* In place, every 128-column block of every row of x [rows, cols] (one attention head of one token):
 * x <- rnd(x / sqrt(mean(x^2) + eps)).  cols a multiple of 128.  Pass the q and k columns of a fused qkv buffer. */
int i8f_rmsnorm_heads(void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ldx, float eps, void* stream);

/* Quantisation with one scale for the whole tensor (weights).
 *   scale_out[0] = max(absmax(x)/127, 1e-30); q as above.
 * `scratch` is 4 bytes of device memory owned by the caller (absmax exchange).
 * hadamard128 rotates each row block in fp32 first (any x_dtype; values are converted to fp32).
 * Replaces quantize_int8_tensorwise (int8_quant.py:23-26) and rotate_weight
 * (quarot.py:42-70). */
int i8f_quant_tensorwise(const void* x, int x_dtype, int64_t N, int64_t K, int64_t ldx,
                         int8_t* q, int64_t ldq, float* scale_out, int hadamard128,
                         void* scratch, void* stream);

/* Per-output-channel weight quantisation (on-the-fly load path).
 *   w [N,K] (w_dtype) -> q int8 [N,K], scale fp32 [N]; values are converted to
 * fp32 first, hadamard128 rotates in fp32 (no intermediate rounding).
 * Replaces int8_quant.py:597-613. */
int i8f_quant_weight_rows(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw,
                          int8_t* q, int64_t ldq, float* scale, int hadamard128, void* stream);

/* Exact int32 = a [M,K] (int8) x w [N,K]^T (int8) on the tcgen05 tensor cores.
 * Replaces torch._int_mm at int8_quant.py:80, :110 (parity / debugging entry). */
int i8f_gemm_i8_i32(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw,
                    int32_t* acc, int64_t ldacc, int64_t M, int64_t N, int64_t K, void* stream);

/* Quantised linear from already quantised activations:
 *   out[m,n] = dequant(sum_k a[m,k] w[n,k]) (+ bias[n])
 * a_scale fp32 [M]; w_scale fp32 [1] or [N] per w_scale_mode; bias (may be
 * NULL) [N] in bias_dtype; out [M,N] in out_dtype (I8F_BF16 or I8F_F16).
 * epilogue_order selects I8F_EPI_PYTORCH (int8_quant.py:84-88, :115-119) or
 * I8F_EPI_SINGLE (int8_fused_kernel.py:146-173, :302-324).
 * Replaces _int8_matmul_dequant_kernel / _per_row (int8_fused_kernel.py:91-173, :253-324). */
int i8f_linear_w8a8(const int8_t* a, int64_t lda, const float* a_scale,
                    const int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode,
                    const void* bias, int bias_dtype,
                    void* out, int out_dtype, int64_t ldo,
                    int64_t M, int64_t N, int64_t K, int epilogue_order, void* stream);

/* Same as i8f_linear_w8a8, then adds what `out` held on entry:
 *   out = round(round(dequant (+bias)) + out_before)
 * With out_before = round(t @ lora_b^T) from i8f_lora_up this is the dynamic-LoRA forward
 * y + lora_y.to(y.dtype) of int8_quant.py:763-774 with the same three roundings, and the read of the
 * LoRA term overlaps the tensor-core main loop instead of costing a separate pass over y. */
int i8f_linear_w8a8_add(const int8_t* a, int64_t lda, const float* a_scale,
                        const int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode,
                        const void* bias, int bias_dtype,
                        void* out, int out_dtype, int64_t ldo,
                        int64_t M, int64_t N, int64_t K, int epilogue_order, void* stream);

/* Gated residual update in the epilogue, in place:
 *   out = round(out_before + gate[n] * round(dequant (+bias)))       (reference rounding order for the linear itself)
 * gate [N] in out_dtype.  gate * y is exact in fp32, so the sum has one fp32 rounding before the rounding to
 * out_dtype: the arithmetic of torch.addcmul(out_before, gate, linear(x)), which is how a diffusion transformer
 * block adds a gated branch to its residual stream.  No counterpart in the reference (the model does this step). */
int i8f_linear_w8a8_gated_add(const int8_t* a, int64_t lda, const float* a_scale,
                              const int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode,
                              const void* bias, int bias_dtype, const void* gate,
                              void* out, int out_dtype, int64_t ldo,
                              int64_t M, int64_t N, int64_t K, void* stream);

/* Quantised linear with the dynamic-LoRA term fused in:
 *   out = round(round(dequant (+bias)) + round(t [M,r] @ lora_b [N,r]^T))
 * t and lora_b are in out_dtype (bf16 or fp16), pitches multiples of 8 elements.  The low-rank product is
 * accumulated by the tensor cores in a second (fp32) tensor-memory accumulator next to the int32 one, from
 * operands that ride the same TMA ring as the int8 tiles; the sum never goes through global memory.
 * Replaces the dequant epilogue plus int8_quant.py:769-774 (t comes from i8f_lora_down, :768). */
int i8f_linear_w8a8_lora(const int8_t* a, int64_t lda, const float* a_scale,
                         const int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode,
                         const void* bias, int bias_dtype,
                         const void* t, int64_t ldt, const void* lora_b, int64_t ldb, int64_t r,
                         void* out, int out_dtype, int64_t ldo,
                         int64_t M, int64_t N, int64_t K, int epilogue_order, void* stream);

/* Column-parallel form: computes this GPU's [M,N] block of a wider output (N = n_total / P output channels)
 * and stores it at column `col_offset` of n_dests destination matrices [M, n_total] (pitch ld_dest), which are
 * this GPU's and its peers' copies of the full output (peer pointers mapped into this process, e.g. CUDA IPC or
 * symmetric memory).  The tiles leave the epilogue as TMA stores to every destination, so the all-gather of a
 * column-parallel linear overlaps the tensor-core main loop instead of following it.  No load ever touches peer
 * memory.  The caller orders the peers (a barrier after the kernel) before anyone reads its copy.
 * N must be a multiple of 32; n_dests <= 8.  Has no counterpart in the reference, which is single-GPU. */
int i8f_linear_w8a8_scatter(const int8_t* a, int64_t lda, const float* a_scale,
                            const int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode,
                            const void* bias, int bias_dtype,
                            void* const* dests, int n_dests, int64_t ld_dest, int64_t n_total, int64_t col_offset,
                            int out_dtype, int64_t M, int64_t N, int64_t K, int epilogue_order, void* stream);

/* Meeting point of the ranks of a column-parallel linear (one process per GPU), enqueued on `stream`.
 * flag_arrays[p] is rank p's array of n_ranks 32-bit flags as mapped into THIS process (symmetric memory or
 * CUDA IPC; zero before the first meeting).  The kernel publishes `epoch` in slot `rank` of every array with
 * system-scope stores, then polls its OWN array until every slot has reached `epoch` (compared modulo 2^32, so
 * epochs simply count up and flags are never cleared).  No load touches peer memory.  The wait gives up after
 * `limit_cycles` SM clocks (2e9 is about a second) and records 105 in the device status word, so a rank that
 * failed on the host costs its peers a bounded delay and an error, never a GPU that spins for ever.
 * Ranks must not share a GPU.  n_ranks <= 8.  Has no counterpart in the reference, which is single-GPU. */
int i8f_peer_barrier(void* const* flag_arrays, int n_ranks, int rank, uint32_t epoch, int64_t limit_cycles, void* stream);

/* Bytes of caller-owned workspace i8f_linear_forward needs for an [M,K] input. */
size_t i8f_linear_workspace_bytes(int64_t M, int64_t K);

/* Whole forward of one quantised linear: (rotate) -> per-token quantise ->
 * int8 GEMM -> dequant (+bias) -> out.  `workspace` holds the int8 activations
 * and their scales between the two kernels.
 * Replaces triton_int8_linear / triton_int8_linear_per_row
 * (int8_fused_kernel.py:179-235, :330-372) and the body of
 * int8_forward_dynamic[_per_row] (int8_quant.py:67-119). */
int i8f_linear_forward(const void* x, int x_dtype, int64_t ldx, int hadamard128,
                       const int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode,
                       const void* bias, int bias_dtype,
                       void* out, int out_dtype, int64_t ldo,
                       int64_t M, int64_t N, int64_t K, int epilogue_order,
                       void* workspace, size_t workspace_bytes, void* stream);

/* Size of the workspace built into the library for i8f_linear_forward_static. */
#define I8F_STATIC_WORKSPACE_BYTES (16u * 1024u * 1024u + 256u * 1024u)

/* i8f_linear_forward without a workspace argument, for callers that may not allocate device
 * memory (a host that owns the whole device through its own pool, a loop that must stay off
 * the allocator, a sandbox that may only launch on a given stream).  Same arithmetic and
 * results as i8f_linear_forward; the int8 activations and their scales go to an array that is
 * part of the library image instead.  The call itself requests no memory (no cudaMalloc, no pool).
 *   - Limit: i8f_linear_workspace_bytes(M, K) <= I8F_STATIC_WORKSPACE_BYTES (e.g. M*K up to
 *     4096 x 4096); larger problems return I8F_ERR_WORKSPACE and launch nothing.
 *   - The array exists once per GPU that uses this entry point and stays until the process exits.
 *     With CUDA's default lazy module loading the driver gives the array its device memory when the
 *     module is first touched, which is the FIRST call of this function on a device: device memory in
 *     use grows by the array's size during that call, and it can fail with I8F_ERR_CUDA if nothing is
 *     left.  A host that hands the rest of the GPU to its own pool makes this first call before it does.
 *   - All calls share it: calls that may overlap on the GPU (different streams without an
 *     ordering between them) race.  It keeps the previous call's contents; no part of it
 *     needs to be zero on entry, every byte a call reads it has written first.
 *   - The first call on a device resolves the array's device address; make it before any
 *     stream capture begins.
 * This entry point has no counterpart in the reference (which always allocates through PyTorch). */
int i8f_linear_forward_static(const void* x, int x_dtype, int64_t ldx, int hadamard128,
                              const int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode,
                              const void* bias, int bias_dtype,
                              void* out, int out_dtype, int64_t ldo,
                              int64_t M, int64_t N, int64_t K, int epilogue_order, void* stream);

/* Linear for M <= 16 rows without activation quantisation (the tiny-batch branch of the Linear):
 *   out [M,N] = round(x [M,K] @ dt(fp32(w) * w_scale)^T + dt(bias)),  dt = x_dtype (I8F_BF16 or I8F_F16),
 * one pass over the int8 weights (HBM-bound on N*K bytes), fp32 accumulation, out in x_dtype.
 * K and ldw multiples of 16, ldx a multiple of 8 elements, x and w 16-byte aligned; M > 16 returns
 * I8F_ERR_UNSUPPORTED.  Replaces dequantize(weight, w_scale).to(x.dtype) + F.linear at int8_quant.py:756-760
 * (which materialises the 16-bit weight matrix on every call). */
int i8f_linear_w8a16_small(const void* x, int x_dtype, int64_t ldx,
                           const int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode,
                           const void* bias, int bias_dtype,
                           void* out, int64_t ldo,
                           int64_t M, int64_t N, int64_t K, void* stream);

/* Dynamic-LoRA down projection: t [M,r] = round(x [M,K] @ lora_a [r,K]^T) in
 * `dtype` (I8F_BF16 or I8F_F16; x, lora_a and t share it), fp32 accumulation.
 * Replaces F.linear(x_2d, lora_A) at int8_quant.py:768. */
int i8f_lora_down(const void* x, int64_t ldx, const void* lora_a, int64_t lda,
                  void* t, int64_t ldt, int dtype, int64_t M, int64_t K, int64_t r, void* stream);

/* Dynamic-LoRA up projection alone: y [M,N] = round(t [M,r] @ lora_b [N,r]^T) in `dtype`.
 * Replaces F.linear(lora_x, lora_B) at int8_quant.py:769; feed the result to i8f_linear_w8a8_add. */
int i8f_lora_up(const void* t, int64_t ldt, const void* lora_b, int64_t ldb,
                void* y, int64_t ldy, int dtype, int64_t M, int64_t N, int64_t r, void* stream);

/* Dynamic-LoRA up projection and add: y [M,N] = round(y + round(t [M,r] @ lora_b [N,r]^T)).
 * Replaces int8_quant.py:769-774. */
int i8f_lora_up_add(const void* t, int64_t ldt, const void* lora_b, int64_t ldb,
                    void* y, int64_t ldy, int dtype, int64_t M, int64_t N, int64_t r, void* stream);

/* Stochastic-rounding merge of a low-rank update into int8 weights, in place:
 *   delta = (up [N,r] @ down [r,K]) * lora_scale            (fp32, j ascending)
 *   hadamard128: delta <- delta rotated per 128-block of K   (fp32)
 *   d8    = clamp(floor(delta/ws) + [u < frac], -128, 127)
 *   w     = clamp(int32(w) + d8, -128, 127)
 * ws = w_scale[0] or w_scale[n] per w_scale_mode.  u comes from `uniforms`
 * (fp32 [N,K], pitch K) when non-NULL, else from Philox4x32-10 keyed by
 * `seed` with counter (n, k/8): weight k takes 16-bit half (k%8)%2 (low half first) of word (k%8)/2,
 * u = half * 2^-16 (one generator block serves eight weights).
 * factor_dtype is the dtype of up and down.
 * Replaces reconstruct_lora_diff (plain LoRA, int8_quant.py:139-155),
 * stochastic_round_int8_delta (:36-62) and the add/clamp at :313-316. */
int i8f_lora_merge_sr(int8_t* w, int64_t ldw, const float* w_scale, int w_scale_mode,
                      const void* up, int64_t ldup, const void* down, int64_t lddown, int factor_dtype,
                      int64_t N, int64_t K, int64_t r, float lora_scale, int hadamard128,
                      const float* uniforms, uint64_t seed, void* stream);

/* Largest rank r one i8f_lora_merge_sr launch accepts for contiguous factors of `factor_dtype`
 * (with_uniforms != 0: the call supplies its own uniforms).  A CTA keeps the whole [r x 128] slice of `down`
 * in shared memory, which is what sets the limit: 319 for fp32 factors or supplied uniforms, 576 for 16-bit
 * factors with the in-kernel counter RNG.  Callers with a larger (stacked) rank build the fp32 delta
 * themselves and use i8f_stochastic_round, which has no rank in it.  The reference sums any number of
 * deltas at any rank (int8_quant.py:355-404); the host layer of this package does the same on top of the
 * two entry points. */
int64_t i8f_lora_merge_max_rank(int factor_dtype, int with_uniforms);

/* Stochastic rounding of an existing fp32 delta (same arithmetic as above
 * from `delta/ws` on), written to d8 without touching any weight.
 * Replaces stochastic_round_int8_delta (int8_quant.py:36-62) for callers that
 * already hold the delta (set_weight, :678-680; LoHa/LoKr deltas). */
int i8f_stochastic_round(const float* delta, int64_t ldd, const float* w_scale, int w_scale_mode,
                         int8_t* d8, int64_t ldq, int64_t N, int64_t K,
                         const float* uniforms, uint64_t seed, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* I8F_H_ */
