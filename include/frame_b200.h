/*
 * frame_b200.h — C ABI of libframe_b200.so: hand-written sm_100a (B200) kernels and the CUDA
 * HAL plumbing for the compiled-graph inference path of the Frame deep-learning framework.
 *
 * The library owns no Frame types.  Every entry point takes plain pointers, int64 sizes and a
 * CUDA stream handle, allocates nothing unless its name says so, enqueues on the given stream
 * and returns an fb200_status.  fb200_last_error() returns a thread-local English message for
 * the last non-zero status.  There is no CPU fallback: on a machine without a usable B200 the
 * compute entry points return FB200_DEVICE_ERROR.
 *
 * Each declaration cites the interface of the reference project it stands behind
 * (file:line, paths inside the reference project).  The C++20 adapter that implements
 * hal::Backend / Allocator / Stream / Event / Executable and registers one KernelFn per op
 * with FRAME_REGISTER_KERNEL is the only intended caller inside a Frame process.
 */
#ifndef FRAME_B200_H_
#define FRAME_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FB200_API __attribute__((visibility("default")))
#else
#define FB200_API
#endif

/* Status codes: same numbering as frame::ErrorCode (include/frame/core/status.h:18-27). */
typedef enum fb200_status {
  FB200_OK = 0,
  FB200_INVALID_ARGUMENT = 1,
  FB200_NOT_FOUND = 2,
  FB200_ALREADY_EXISTS = 3,
  FB200_UNIMPLEMENTED = 4,
  FB200_OUT_OF_MEMORY = 5,
  FB200_INTERNAL = 6,
  FB200_DEVICE_ERROR = 7
} fb200_status;

/* Element types: same numbering as frame::DTypeCode (include/frame/core/dtype.h:17-29).
 * bf16/f16 are 16-bit storage PODs (dtype.h:38-43). */
typedef enum fb200_dtype {
  FB200_F32 = 0,
  FB200_F64 = 1,
  FB200_F16 = 2,
  FB200_BF16 = 3,
  FB200_I8 = 4,
  FB200_I16 = 5,
  FB200_I32 = 6,
  FB200_I64 = 7,
  FB200_U8 = 8,
  FB200_BOOL = 9
} fb200_dtype;

/* A cudaStream_t passed as an opaque pointer (hal::Stream::native_handle,
 * include/frame/hal/stream.h:22-28).  NULL = the default stream
 * (ops::KernelContext::stream may be null, include/frame/ops/kernel_registry.h:30-43). */
typedef void* fb200_stream;
typedef void* fb200_event;

/* ---- library ----------------------------------------------------------------------------- */
FB200_API const char* fb200_last_error(void);
FB200_API const char* fb200_version(void);
/* Number of kernels this library has launched in the calling process (for harness accounting). */
FB200_API int64_t fb200_launch_count(void);

/* Reads and clears the per-device kernel status word.  Every wait inside the tensor-core
 * kernels is bounded; a wait that gives up records a non-zero code here and the kernel exits
 * cleanly (its results are then invalid).  0 = healthy.  Read after a stream synchronise. */
FB200_API int fb200_kernel_status(int device, int* code);

/* ---- HAL: devices, allocator, copies, streams, events -------------------------------------
 * Behind hal::Backend::device_count / allocator / copy / create_stream / create_event
 * (include/frame/hal/backend.h:77-109) and hal::Allocator (include/frame/hal/allocator.h:13-21);
 * replaces src/backends/cuda/cuda_backend.cpp:68-312 and cuda_allocator.cpp:26-66. */
FB200_API int fb200_device_count(int* count);
/* PCI bus id of CUDA device `device` as text (at least 16 bytes): the key under which NVML and
 * nvidia-smi know the same physical GPU (their indices ignore CUDA_VISIBLE_DEVICES).  The
 * reference has no counterpart (include/frame/core/device.h:19-24 carries an ordinal only). */
FB200_API int fb200_device_pci_bus_id(int device, char* buf, int len);
/* bytes > 0, alignment a power of two <= 256 (cuda_allocator.cpp:26-41). */
FB200_API int fb200_malloc(int device, size_t bytes, size_t alignment, void** ptr);
FB200_API int fb200_free(int device, void* ptr);
/* Pinned host staging memory for the harness-side end-to-end path. */
FB200_API int fb200_host_alloc(size_t bytes, void** ptr);
FB200_API int fb200_host_free(void* ptr);
typedef enum fb200_copy_kind { FB200_H2D = 1, FB200_D2H = 2, FB200_D2D = 3 } fb200_copy_kind;
/* stream == NULL with blocking != 0 is a synchronous copy (cuda_backend.cpp:194-203);
 * bytes == 0 is a no-op; a null pointer with bytes > 0 is FB200_INVALID_ARGUMENT. */
FB200_API int fb200_memcpy(int device, void* dst, const void* src, size_t bytes, int kind,
                           fb200_stream stream, int blocking);
FB200_API int fb200_memset(int device, void* dst, int value, size_t bytes, fb200_stream stream);
FB200_API int fb200_stream_create(int device, fb200_stream* stream);
FB200_API int fb200_stream_destroy(int device, fb200_stream stream);
FB200_API int fb200_stream_synchronize(int device, fb200_stream stream);
FB200_API int fb200_event_create(int device, int timing, fb200_event* event);
FB200_API int fb200_event_destroy(int device, fb200_event event);
FB200_API int fb200_event_record(int device, fb200_event event, fb200_stream stream);
FB200_API int fb200_stream_wait_event(int device, fb200_stream stream, fb200_event event);
/* *done = 1 when complete (include/frame/hal/event.h:16-24). */
FB200_API int fb200_event_query(int device, fb200_event event, int* done);
FB200_API int fb200_event_synchronize(int device, fb200_event event);
FB200_API int fb200_event_elapsed_ms(fb200_event start, fb200_event stop, float* ms);

/* ---- elementwise and fused groups ----------------------------------------------------------
 * Sub-op codes of a fused elementwise chain.  add/mul/relu/square/sigmoid/tanh/rsqrt follow
 * src/backends/cpu/kernels/elementwise.cpp:39-56,146-163,242-255,329-404; gelu (tanh form),
 * silu, softplus, exp have no counterpart in the reference (new ops). */
typedef enum fb200_ew_op {
  FB200_EW_ADD = 1,
  FB200_EW_MUL = 2,
  FB200_EW_RELU = 3,
  FB200_EW_SQUARE = 4,
  FB200_EW_SIGMOID = 5,
  FB200_EW_TANH = 6,
  FB200_EW_RSQRT = 7,
  FB200_EW_GELU = 8,
  FB200_EW_SILU = 9,
  FB200_EW_SOFTPLUS = 10,
  FB200_EW_EXP = 11,
  FB200_EW_HEAVISIDE = 12,  /* heaviside_surrogate forward: x >= 0 ? 1 : 0 (src/backends/cpu/kernels/elementwise.cpp, heaviside_surrogate_cpu_kernel) */
  FB200_EW_RELU_GRAD = 13   /* relu_grad_internal(x, gy): x > 0 ? gy : 0, binary and NOT commutative: the running value is x, the operand gy (elementwise.cpp:411-414); elementwise chains only, not a matmul / conv2d epilogue step */
} fb200_ew_op;
#define FB200_MAX_CHAIN 8
#define FB200_MAX_CHAIN_INPUTS 9

/* One launch for a whole fused group: op `fused_elementwise_internal` with attrs
 * ops="add;mul;relu", arities=[2,2,1] (include/frame/ops/fused_elementwise_utils.h:28,44-59).
 * Wiring as src/ops/fused_elementwise_utils.cpp:88-101,141-165: segment 0 reads its operands
 * from `inputs`; segment i>0 takes the previous result as operand 0 and the next external
 * inputs for the rest.  Every intermediate is rounded to `dtype` exactly as the unfused chain
 * does.  A chain of one op is the standalone op (elementwise.cu:582-785 of the reference CUDA
 * backend).  dtype: F32, BF16, F16; I32/I64 for a chain consisting of `add` only. */
FB200_API int fb200_fused_elementwise(const void* const* inputs, int n_inputs, void* out,
                                      int64_t numel, int dtype, const int* ops,
                                      const int* arities, int n_ops, fb200_stream stream);
/* NEW op: out[r, j] = x[r, j] + bias[j] (row-broadcast bias; no reference counterpart, the
 * reference only has same-shape add, src/ops/schemas/elementwise.cpp:41-66). */
FB200_API int fb200_bias_add(const void* x, const void* bias, void* out, int64_t rows,
                             int64_t cols, int dtype, fb200_stream stream);

/* ---- epilogue shared by matmul and conv2d --------------------------------------------------
 * A short elementwise chain applied to the accumulator before the single store.  Binary steps
 * read a second operand: same shape as the output (mode FULL, what reference graphs contain:
 * a Linear bias is a full [batch,out] tensor, src/nn/layers.cpp:241-248), one value per output
 * column (mode COL: matmul [N]; conv2d: unused) or one value per output row / channel
 * (mode ROW: conv2d per-Cout). */
typedef enum fb200_operand_mode { FB200_OPERAND_FULL = 0, FB200_OPERAND_COL = 1, FB200_OPERAND_ROW = 2 } fb200_operand_mode;
typedef struct fb200_epilogue {
  int n_ops;
  int ops[FB200_MAX_CHAIN];
  const void* operands[FB200_MAX_CHAIN]; /* NULL for unary steps */
  int modes[FB200_MAX_CHAIN];
} fb200_epilogue;

/* ---- dense contractions --------------------------------------------------------------------
 * matmul: C[m,n] = sum_p A[m,p]*B[p,n], rank-2 row-major operands of one dtype, fp32
 * accumulation, one rounding at the store (src/backends/cpu/kernels/matmul.cpp:92-131;
 * replaces the cublasLtMatmul call of src/backends/cuda/kernels/matmul.cpp:90-276).
 * BF16/F16: tcgen05 kind::f16.  F32: allow_tf32 != 0 selects tcgen05 kind::tf32 (the
 * CompileOptions::allow_tf32 switch, include/frame/hal/backend.h:51-63); allow_tf32 == 0 keeps
 * fp32 accuracy: products below 2^30 multiply-adds (and shapes TMA cannot address) run on the CUDA
 * cores in the CPU reference's order of additions (bit-identical to it); larger ones run on the
 * tensor cores as three TF32 products with the operands' low parts (error-compensated "3xTF32":
 * no operand rounding left; the tensor core truncates its fp32 accumulator at each of the K/8
 * additions, which leaves about 2^-23 * K/8 of the result's scale: 5-30 times a round-to-nearest
 * fp32 summation, 50-100 times below TF32; about a third of the TF32 rate).  allow_tf32 < 0 forces the CPU's order at any
 * size.  `epilogue` may be NULL. */
FB200_API int fb200_matmul(const void* a, const void* b, void* c, int64_t m, int64_t n,
                           int64_t k, int dtype, int allow_tf32, const fb200_epilogue* epilogue,
                           fb200_stream stream);
/* The same product leaving in two pieces: columns [0, tail_col) go to `c` exactly where fb200_matmul
 * puts them (row pitch n; the columns from tail_col on stay untouched there), columns
 * [tail_col, n) go to the dense matrix `c_tail` [m, n - tail_col].  Replaces the reference's
 * matmul followed by a `slice` of that column block (src/backends/cuda/kernels/shape.cpp:207, one
 * cudaMemcpyAsync per row): the block is stored once, where the slice would have copied it.
 * tail_col: a multiple of 32 in (0, n); tensor-core shapes only (fb200_matmul_uses_tensor_cores). */
FB200_API int fb200_matmul_split(const void* a, const void* b, void* c, void* c_tail, int64_t tail_col,
                                 int64_t m, int64_t n, int64_t k, int dtype, int allow_tf32,
                                 const fb200_epilogue* epilogue, fb200_stream stream);
/* Which kernel family fb200_matmul would pick: 1 = tcgen05/TMEM/TMA, 0 = SIMT. */
FB200_API int fb200_matmul_uses_tensor_cores(int64_t m, int64_t n, int64_t k, int dtype,
                                             int allow_tf32);
/* How fb200_matmul would schedule a tensor-core product (no reference counterpart: cuBLASLt keeps
 * its heuristics to itself).  out6 = {tile columns, tile rows, tiles walked whole, k-blocks dealt
 * out in ranges, CTAs taking a range, k-blocks per tile}.  When a few tiles (a quarter of the SMs or
 * fewer) carry a long K (128 k-blocks of 128 bytes or more: the weight-gradient shape), their
 * k-blocks are split into equal contiguous ranges over the SMs ("stream-K"): the CTA holding a
 * tile's first k-blocks adds the partial accumulators of the ranges after it, in range order
 * (results do not depend on timing), and runs the epilogue.  A CTA only waits for CTAs that started
 * before it (ranges are handed out against a ticket taken at entry), so such launches need no
 * co-residency guarantee and every wait is bounded; their
 * partial-tile scratch (19 MB) is kept per stream.  light_epilogue_chain: the chain is adds, multiplies and ReLU only;
 * compensated: the three-pass strict fp32 form. */
FB200_API int fb200_matmul_schedule(int64_t m, int64_t n, int64_t k, int dtype, int light_epilogue_chain,
                                    int compensated, int64_t* out6);

/* Column-split matmul with the all-gather of C fused into the epilogue (the optional multi-GPU
 * variant of the GEMM config; the reference has no multi-GPU code at all).  This rank computes
 * epilogue(A . B_local) for its column block [col0, col0+n_local) and stores it into that block of
 * every matrix in c_dest (row pitch n_total): its own C and its peers' copies, imported with
 * fb200_ipc_import.  Peer stores are plain global stores over NVLink; after a stream synchronise
 * and a host-side barrier every GPU holds the whole C.  Epilogue operands use the local
 * [m, n_local] layout. */
FB200_API int fb200_matmul_colsplit(const void* a, const void* b_local, void* const* c_dest,
                                    int n_dest, int64_t m, int64_t n_local, int64_t n_total,
                                    int64_t col0, int64_t k, int dtype, int allow_tf32,
                                    const fb200_epilogue* epilogue, fb200_stream stream);
/* CUDA IPC handles (64 bytes) for device allocations, to map a peer process's buffer. */
FB200_API int fb200_ipc_export(int device, void* ptr, void* handle64);
FB200_API int fb200_ipc_import(int device, const void* handle64, void** ptr);
FB200_API int fb200_ipc_close(int device, void* ptr);

/* conv2d: NCHW cross-correlation with groups, stride, zero padding, optional [Cout] bias,
 * accumulation in fp32 (src/backends/cpu/kernels/conv.cpp:225-257; schema
 * src/ops/schemas/conv.cpp:979-989; replaces cudnnConvolutionForward,
 * src/backends/cuda/kernels/conv.cpp:385-520). */
typedef struct fb200_conv2d_params {
  int64_t n, cin, h, w;
  int64_t cout, kh, kw;
  int64_t stride_h, stride_w, pad_h, pad_w, groups;
} fb200_conv2d_params;
FB200_API int fb200_conv2d(const void* x, const void* w, const void* bias, void* out,
                           const fb200_conv2d_params* p, int dtype, int allow_tf32,
                           const fb200_epilogue* epilogue, fb200_stream stream);
/* conv1d: NCL, same conventions (src/backends/cpu/kernels/conv.cpp:565-589; the reference CUDA
 * backend has no kernel for it and falls back, src/ops/schemas/conv.cpp:1021-1032). */
FB200_API int fb200_conv1d(const void* x, const void* w, const void* bias, void* out, int64_t n,
                           int64_t cin, int64_t l, int64_t cout, int64_t k, int64_t stride,
                           int64_t padding, int64_t groups, int dtype, fb200_stream stream);
/* Depthwise conv1d along time in the TIME-MAJOR layout, with trailing unary elementwise ops.
 * Stands behind the five-step group transpose [B,L,C]->[B,C,L], conv1d(groups = C), slice,
 * activation, transpose back of the reference's Mamba block (src/nn/layers.cpp:1596-1602; conv1d:
 * src/backends/cpu/kernels/conv.cpp:565-589), with the same operations in the same order:
 *   out[b,t,c] = ops(bias[c] + sum_k w[c,k] * x[b, t+shift+k, c]),  taps outside [0, len) skipped,
 * shift = slice_start - padding (-(k-1) for the causal form).  x: [batch, len] rows of pitch x_ld
 * (a column window of a wider matrix works), out: [batch, out_len] rows of pitch out_ld, w: [C,1,k],
 * bias: [C] or NULL.  channels and both pitches must be multiples of the 16-byte vector width;
 * 1 <= k <= 8; unary_ops: FB200_EW_* codes applied in order, each rounded to the dtype. */
FB200_API int fb200_dwconv1d_time_major(const void* x, int64_t x_ld, const void* w, const void* bias,
                                        void* out, int64_t out_ld, int64_t batch, int64_t len,
                                        int64_t out_len, int64_t channels, int64_t k, int64_t shift,
                                        const int* unary_ops, int n_ops, int dtype,
                                        fb200_stream stream);
/* avg_pool2d: sum over the valid positions of the window in (kh, kw) order divided by KH*KW
 * (padding counts in the denominator), src/backends/cpu/kernels/pool.cpp:280-303; replaces
 * cudnnPoolingForward of src/backends/cuda/kernels/pool.cpp.  Same geometry rules as max_pool2d. */
FB200_API int fb200_avg_pool2d(const void* x, void* out, int64_t n, int64_t c, int64_t h,
                               int64_t w, int64_t kh, int64_t kw, int64_t stride_h,
                               int64_t stride_w, int64_t pad_h, int64_t pad_w, int dtype,
                               fb200_stream stream);
/* Gradient-side internals of pooling and convolution (n, c, h, w and the params describe the FORWARD
 * op's input x; out_h = (h + 2*pad_h - kh) / stride_h + 1, likewise out_w).  All are computed as
 * gathers over their output, in the CPU reference's operation order: fp32 results are bit-identical.
 *  max_pool2d_select_internal: out[n,c,oh,ow] = g[n,c, argmax of x over the window] (first maximum,
 *    strict >), g and x [n,c,h,w]; src/backends/cpu/kernels/pool.cpp:459-483.
 *  max_pool2d_grad_internal: dx [n,c,h,w] = dy [n,c,oh,ow] added into each window's argmax of x,
 *    windows in (oh, ow) order; pool.cpp:356-389 (replaces cudnnPoolingBackward).
 *  avg_pool2d_grad_internal: dx[n,c,ih,iw] = (sum of dy over the windows that cover it) / (KH*KW);
 *    pool.cpp:542-568.
 *  conv2d_grad_input_internal: dx [n,cin,h,w] from dy [n,cout,oh,ow] and w [cout,cin/groups,kh,kw],
 *    terms in (co, kh, kw) order; src/backends/cpu/kernels/conv.cpp:321-353 (replaces
 *    cudnnConvolutionBackwardData).
 *  conv2d_grad_filter_internal: dw [cout,cin/groups,kh,kw] from x and dy, terms in (n, oh, ow) order;
 *    conv.cpp:424-453 (replaces cudnnConvolutionBackwardFilter). */
FB200_API int fb200_max_pool2d_select(const void* g, const void* x, void* out, int64_t n, int64_t c,
                                      int64_t h, int64_t w, int64_t kh, int64_t kw, int64_t stride_h,
                                      int64_t stride_w, int64_t pad_h, int64_t pad_w, int dtype,
                                      fb200_stream stream);
FB200_API int fb200_max_pool2d_grad(const void* dy, const void* x, void* dx, int64_t n, int64_t c,
                                    int64_t h, int64_t w, int64_t kh, int64_t kw, int64_t stride_h,
                                    int64_t stride_w, int64_t pad_h, int64_t pad_w, int dtype,
                                    fb200_stream stream);
FB200_API int fb200_avg_pool2d_grad(const void* dy, void* dx, int64_t n, int64_t c, int64_t h,
                                    int64_t w, int64_t kh, int64_t kw, int64_t stride_h,
                                    int64_t stride_w, int64_t pad_h, int64_t pad_w, int dtype,
                                    fb200_stream stream);
FB200_API int fb200_conv2d_grad_input(const void* dy, const void* w, void* dx,
                                      const fb200_conv2d_params* p, int dtype, fb200_stream stream);
FB200_API int fb200_conv2d_grad_filter(const void* x, const void* dy, void* dw,
                                       const fb200_conv2d_params* p, int dtype, fb200_stream stream);
/* Gradients of matmul (src/backends/cpu/kernels/matmul.cpp:187-232, :289-330; the reference CUDA
 * backend has no kernel for them): ga[m,k] = gy[m,n] * b[k,n]^T and gb[k,n] = a[m,k]^T * gy[m,n],
 * fp32 accumulation over the contracted index in increasing order, one rounding.  Strict fp32 reads
 * the transposed operand in place (bit-identical to the CPU reference); bf16 / f16 and fp32 with
 * allow_tf32 transpose it once into a stream-ordered scratch and run the tensor-core GEMM. */
FB200_API int fb200_matmul_grad_lhs(const void* gy, const void* b, void* ga, int64_t m, int64_t n,
                                    int64_t k, int dtype, int allow_tf32, fb200_stream stream);
FB200_API int fb200_matmul_grad_rhs(const void* a, const void* gy, void* gb, int64_t m, int64_t n,
                                    int64_t k, int dtype, int allow_tf32, fb200_stream stream);
/* mse_loss(pred, target) = mean((pred - target)^2) -> one element; mse_loss_grad_internal =
 * (2*gy/numel) * (pred - target) with gy one element (src/backends/cpu/kernels/loss.cpp:108-150,
 * :225-255).  The loss is bit-identical to the serial fp32 sum of the reference up to 65536
 * elements and a double-precision block reduction above; the gradient is bit-identical. */
FB200_API int fb200_mse_loss(const void* pred, const void* target, void* out, int64_t numel,
                             int dtype, fb200_stream stream);
FB200_API int fb200_mse_loss_grad(const void* pred, const void* target, const void* gy, void* gpred,
                                  int64_t numel, int dtype, fb200_stream stream);
/* rfft / irfft along the last axis, float32 only (src/ops/schemas/fft.cpp:8-9; replace the cuFFT
 * R2C / C2R plans of src/backends/cuda/kernels/fft.cpp).  rfft: x [rows, n] -> out [rows, n/2+1, 2]
 * (interleaved re/im, forward sign, unscaled).  irfft: z [rows, n/2+1, 2] -> out [rows, n], scaled by
 * 1/n; the imaginary parts of the DC and (even n) Nyquist terms are ignored.  Direct O(n^2)
 * transforms accumulated in double precision and rounded once. */
FB200_API int fb200_rfft(const void* x, void* out, int64_t rows, int64_t n, int dtype,
                         fb200_stream stream);
FB200_API int fb200_irfft(const void* z, void* out, int64_t rows, int64_t n, int dtype,
                          fb200_stream stream);
/* gather along axis 0: out[k, :] = x[indices[k], :], x [n, f], indices [k] of int32 / int64
 * (src/ops/schemas/gather.cpp:86-118; replaces src/backends/cuda/kernels/gather.cu).  An index
 * outside [0, n) is an error that names the value, found like the reference does by looking at the
 * indices before the copy: this entry point synchronises the stream once for that.
 * scatter_add / gather_grad_internal: out [v, f] = 0, then out[indices[k], :] += updates[k, :]
 * (repeated indices accumulate; fp32 atomics, so the order of additions is not fixed and results
 * agree with the CPU reference within the tolerance tier, not bit for bit). */
FB200_API int fb200_gather(const void* x, const void* indices, void* out, int64_t n, int64_t f,
                           int64_t k, int dtype, int index_dtype, fb200_stream stream);
FB200_API int fb200_scatter_add(const void* updates, const void* indices, void* out, int64_t k,
                                int64_t f, int64_t v, int dtype, int index_dtype,
                                fb200_stream stream);
/* max_pool2d: max over valid positions only, first maximum wins
 * (src/backends/cpu/kernels/pool.cpp:187-233; replaces cudnnPoolingForward,
 * src/backends/cuda/kernels/pool.cpp:231). */
/* conv2d -> [epilogue chain] -> max_pool2d in one call (replaces the reference's three launches for
 * an image stem: cudnnConvolutionForward + cudnnAddTensor, the activation, cudnnPoolingForward:
 * src/backends/cuda/kernels/conv.cpp:385-520, pooling.cpp).  With allow_tf32, a 3x3 / stride 2 /
 * pad 1 pool behind a stride-2 convolution with kw * cin <= 32, 32 < cout <= 64, an even number of
 * output rows of at most 128 pixels and a chain of unary steps runs as ONE kernel that pools the
 * rows in its epilogue and never writes the convolution's result; `mid` ([n, cout, oh, ow]) is then
 * untouched and may be NULL.  Every other case runs fb200_conv2d into `mid` and fb200_max_pool2d. */
FB200_API int fb200_conv2d_max_pool(const void* x, const void* w, const void* bias, void* mid, void* out,
                                    const fb200_conv2d_params* params, int64_t pool_kh, int64_t pool_kw,
                                    int64_t pool_stride_h, int64_t pool_stride_w, int64_t pool_pad_h,
                                    int64_t pool_pad_w, int dtype, int allow_tf32,
                                    const fb200_epilogue* epilogue, fb200_stream stream);
FB200_API int fb200_max_pool2d(const void* x, void* out, int64_t n, int64_t c, int64_t h,
                               int64_t w, int64_t kh, int64_t kw, int64_t stride_h,
                               int64_t stride_w, int64_t pad_h, int64_t pad_w, int dtype,
                               fb200_stream stream);

/* ---- row kernels ---------------------------------------------------------------------------
 * softmax over the last axis of a rank-2 tensor (src/backends/cpu/kernels/sequence.cpp:114-174;
 * replaces cudnnSoftmaxForward, src/backends/cuda/kernels/sequence.cpp:108-174). */
FB200_API int fb200_softmax(const void* x, void* out, int64_t rows, int64_t cols, int dtype,
                            fb200_stream stream);
/* layer_norm over the last axis, gamma/beta of shape [cols], eps cast to float
 * (src/backends/cpu/kernels/sequence.cpp:182-279; replaces
 * src/backends/cuda/kernels/sequence.cu:104-155). */
FB200_API int fb200_layer_norm(const void* x, const void* gamma, const void* beta, void* out,
                               int64_t rows, int64_t cols, double eps, int dtype,
                               fb200_stream stream);
/* layer_norm(x + res): a transformer block's residual add and the normalisation behind it in one
 * pass (the reference runs `add` and `layer_norm` as two launches, src/backends/cuda/kernels/
 * sequence.cpp).  sum_out receives x + res rounded to the dtype, exactly what the separate add
 * stores; out the normalised rows.  Shapes outside the vector path run as the two operators. */
FB200_API int fb200_add_layer_norm(const void* x, const void* res, const void* gamma, const void* beta,
                                   void* sum_out, void* out, int64_t rows, int64_t cols, double eps,
                                   int dtype, fb200_stream stream);
/* selective_scan: per row h_t = a_t*h_{t-1} + b_t*x_t, y_t = c_t*h_t + d_t*x_t, h_{-1} = 0,
 * time on the last axis, fp32 state (src/backends/cpu/kernels/sequence.cpp:95-106; replaces the
 * per-row CUB scans of src/backends/cuda/kernels/sequence.cu:170-217).  One launch. */
FB200_API int fb200_selective_scan(const void* x, const void* a, const void* b, const void* c,
                                   const void* d, void* out, int64_t rows, int64_t steps,
                                   int dtype, fb200_stream stream);
/* selective_scan that allocates nothing (no counterpart in the reference: its CUDA path allocates
 * scratch with cudaMalloc on every call, src/backends/cuda/kernels/sequence.cu:173-186).  For hosts
 * that must not allocate device memory while the op runs — work being captured into a CUDA graph, or
 * a process that planned all of its device memory up front.  Same results as fb200_selective_scan's
 * chunked two-pass path; its scratch is a fixed 512 KiB array inside the library image (held by
 * every GPU that loads the library until the process exits), good for rows <= 65536; more rows are
 * rejected with FB200_INVALID_ARGUMENT.  Needs 16-byte aligned operands and steps a multiple of the
 * 128-bit vector width.  The first call on a device looks up the array's address on that device
 * (make that call before starting a stream capture, with the device current).  All calls share
 * the one array (every entry is rewritten by a call before it is read, nothing needs clearing), so
 * two calls that overlap on the GPU — different streams, or graphs replayed concurrently — race. */
FB200_API int fb200_selective_scan_noalloc(const void* x, const void* a, const void* b,
                                           const void* c, const void* d, void* out, int64_t rows,
                                           int64_t steps, int dtype, fb200_stream stream);
/* A fan of per-head attention chains in one launch.  Stands behind the per-(batch, head) node
 * groups `matmul(q, transpose(k)) -> softmax -> matmul(p, v)` that the reference builds in
 * nn::MultiHeadAttention (src/nn/layers.cpp:950-1170) and runs node by node
 * (src/backends/cuda/cuda_executable.cpp:84-118).  The scores and the result are rounded to the
 * storage dtype where the separate operators round them; the probabilities are rounded before the
 * division by their row sum, which is applied in fp32 to the second product (the separate softmax
 * rounds the quotient): one rounding per probability either way.  O_h must not overlap any Q, K
 * or V window that another head or query block still reads.  For head h:
 *   Q_h = sq x 64 window of q_base (row-major, q_rows x q_ld) at (q_row, q_col); K_h, V_h likewise
 *   with sk rows; O_h (sq x 64, row pitch o_ld) is written at element offset o_offset of o_base.
 * `scale` (> 0; 1 = none) stands for the elementwise `mul` by a constant that the reference's
 * attention puts between the first matmul and the softmax (src/nn/layers.cpp:1062-1071): the
 * rounded scores are multiplied by it and rounded to the storage dtype again (a power of two
 * multiplies bfloat16 scores exactly and is folded into the exponent instead).
 * Column coordinates must be multiples of 8 elements (a table entry that is not is refused by
 * the kernel, which records status 305).  `heads_dev` is a DEVICE array owned by the caller.
 * Supported: bfloat16 / float16, head_dim 64, 64 <= sk <= 512 in multiples of 64, any sq >= 1
 * (fb200_attention_fan_supported tells); anything else returns FB200_UNIMPLEMENTED. */
typedef struct fb200_attention_head {
  int32_t q_row, q_col, k_row, k_col, v_row, v_col;
  int64_t o_offset;
} fb200_attention_head;
FB200_API int fb200_attention_fan_supported(int64_t sq, int64_t sk, int64_t head_dim, int dtype);
FB200_API int fb200_attention_fan(const void* q_base, int64_t q_rows, int64_t q_ld,
                                  const void* k_base, int64_t k_rows, int64_t k_ld,
                                  const void* v_base, int64_t v_rows, int64_t v_ld, void* o_base,
                                  int64_t o_ld, const fb200_attention_head* heads_dev,
                                  int64_t n_heads, int64_t sq, int64_t sk, int64_t head_dim,
                                  float scale, int dtype, fb200_stream stream);
/* NEW op (no reference counterpart): the Mamba SSM scan with un-materialised operands, fp32.
 * u, delta, z, y: [batch, len, dm]; A: [dm, nstate]; B, C: [batch, len, nstate]; D: [dm];
 * z may be NULL.  h[n] = exp(delta*A[d,n])*h[n] + delta*B[n]*u; y = sum_n C[n]*h[n] + D[d]*u;
 * y *= silu(z).  nstate <= 16. */
FB200_API int fb200_mamba_scan(const void* u, const void* delta, const void* A, const void* B,
                               const void* C, const void* D, const void* z, void* y,
                               int64_t batch, int64_t len, int64_t dm, int64_t nstate,
                               fb200_stream stream);

/* ---- data movement -------------------------------------------------------------------------
 * transpose: out.dims[i] = x.dims[perm[i]] (src/ops/schemas/shape.cpp:424-429;
 * src/backends/cpu/kernels/shape.cpp:73; replaces src/backends/cuda/kernels/shape.cu:65-83). */
FB200_API int fb200_transpose(const void* x, void* out, int rank, const int64_t* dims,
                              const int64_t* perm, int itemsize, fb200_stream stream);
/* slice: one half-open range on one axis (shape.cpp:276; replaces the per-segment
 * cudaMemcpyAsync loop of src/backends/cuda/kernels/shape.cpp:342). */
FB200_API int fb200_slice(const void* x, void* out, int rank, const int64_t* dims, int64_t axis,
                          int64_t start, int64_t stop, int itemsize, fb200_stream stream);
/* concat along one axis (shape.cpp:172; replaces src/backends/cuda/kernels/shape.cpp:207).
 * `axis_sizes[i]` is input i's extent on `axis`; `out_dims` is the output shape. */
FB200_API int fb200_concat(const void* const* inputs, int n_inputs, const int64_t* axis_sizes,
                           void* out, int rank, const int64_t* out_dims, int64_t axis,
                           int itemsize, fb200_stream stream);
/* sum over an axis subset (src/backends/cpu/kernels/reduction.cpp:130; replaces
 * src/backends/cuda/kernels/reduction.cu:90-130). */
FB200_API int fb200_sum_axes(const void* x, void* out, int rank, const int64_t* dims,
                             const int64_t* axes, int n_axes, int dtype, fb200_stream stream);

/* ---- whole-plan executor -------------------------------------------------------------------
 * Runs the step list that ops::build_executable_plan produces for the nine-pass pipeline's
 * output (include/frame/ops/executable_plan.h:42-71), honouring the memory planner's arena
 * offsets (src/ir/memory_plan.cpp:37-133).  Replaces CudaExecutable::run
 * (src/backends/cuda/cuda_executable.cpp:41-128): the arena is allocated once per plan, graph
 * outputs are written straight into the caller's buffers, constants are materialised once,
 * reshape is a zero-copy alias, and matmul/conv2d steps absorb a following elementwise group
 * as their epilogue when it is their only consumer.
 *
 * `plan_text` is the line-oriented form written by the reference-side shim
 * (`plan slots= arena=`, `in`, `step`, `attr`, `out` lines). */
typedef struct fb200_plan fb200_plan;
FB200_API int fb200_plan_create(const char* plan_text, int device, int allow_tf32, int opt_level,
                                fb200_plan** plan);
/* The same parsing and rewriting without a device: allocates nothing on the GPU (and needs none),
 * so the result only answers fb200_plan_launches_per_run / fb200_plan_step_op / io_spec /
 * arena_bytes; every run entry point refuses it.  For tooling and for tests of the rewrite rules on
 * machines without a GPU.  allow_tf32 as for fb200_plan_create (some rewrites depend on which
 * matmuls take the tensor-core kernel).  Free it with fb200_plan_destroy. */
FB200_API int fb200_plan_describe(const char* plan_text, int allow_tf32, int opt_level, fb200_plan** plan);
FB200_API int fb200_plan_destroy(fb200_plan* plan);
FB200_API int fb200_plan_num_inputs(const fb200_plan* plan);
FB200_API int fb200_plan_num_outputs(const fb200_plan* plan);
/* dtype, rank and dims (up to 8) of input/output `index`. */
FB200_API int fb200_plan_io_spec(const fb200_plan* plan, int is_output, int index, int* dtype,
                                 int* rank, int64_t* dims);
FB200_API size_t fb200_plan_arena_bytes(const fb200_plan* plan);
/* Bytes of the plan's private buffers, per stream workspace, beside the arena: results that a
 * rewrite moved out of the planner's layout (a matmul's separately stored column block; the result
 * of an attention fan that the planner, laying out the unfused graph, had put over the fan's own
 * source matrices).  No counterpart in the reference. */
FB200_API size_t fb200_plan_private_bytes(const fb200_plan* plan);
/* Number of kernel launches one run enqueues (after epilogue absorption and aliasing). */
FB200_API int fb200_plan_launches_per_run(const fb200_plan* plan);
/* Device pointers in, device pointers out; asynchronous on `stream`.  Every stream that runs the
 * plan gets a workspace of its own (arena at the planner's offsets, private buffers, captured CUDA
 * graphs), up to four: host threads that run one plan on different streams do not wait for one
 * another and their launches overlap on the device (the reference allocates an arena inside every
 * run for the same effect, src/backends/cuda/cuda_executable.cpp:55-61).  Callers that share a stream,
 * and streams beyond the fourth, take turns.  The host-buffer entry points below share one set of
 * staging buffers and are for one caller at a time. */
FB200_API int fb200_plan_run(fb200_plan* plan, const void* const* inputs, void* const* outputs,
                             fb200_stream stream);
/* Host buffers in and out: H2D of every input, the run, D2H of every output, one stream
 * synchronise.  Staging buffers on the device are owned by the plan. */
FB200_API int fb200_plan_run_host(fb200_plan* plan, const void* const* host_inputs,
                                  void* const* host_outputs, fb200_stream stream);
/* The same, pipelined: returns when the work of this run is queued.  Inputs are copied on a copy-in
 * stream, the plan runs on `stream` (must not be NULL), outputs are copied on a copy-out stream; two
 * staging sets alternate, so H2D of run k+1, run k and D2H of run k-1 overlap.  Host outputs of a run
 * are valid after fb200_plan_host_sync; its host inputs must stay unchanged until then.  Use pinned
 * host memory (fb200_host_alloc).  No counterpart in the reference, whose Executable::run takes device
 * tensors and leaves the copies to the caller (include/frame/hal/executable.h:33). */
FB200_API int fb200_plan_run_host_async(fb200_plan* plan, const void* const* host_inputs,
                                        void* const* host_outputs, fb200_stream stream);
FB200_API int fb200_plan_host_sync(fb200_plan* plan);
/* Marks graph input `index` as a parameter that already lives on the device: the two host-buffer
 * entry points above then read `device_ptr` in place and ignore the matching host pointer (NULL
 * restores the copy).  This is how Frame itself runs a module: nn:: parameters, including the
 * full-shape [batch, out] biases of nn::Linear (src/nn/layers.cpp:241-248), are device tensors the
 * caller passes to Executable::run every time (include/frame/hal/executable.h:33); only the
 * activations of a step travel.  The caller keeps the buffer alive while runs are in flight. */
FB200_API int fb200_plan_bind_resident(fb200_plan* plan, int index, const void* device_ptr);

/* Per-step device times (ms) of one eager run, measured with CUDA events on `stream`; steps that
 * launch nothing report 0.  For harness-side accounting of which kernel dominates a graph; has no
 * counterpart in the reference (it has no profiling hooks).  Synchronises the stream. */
FB200_API int fb200_plan_profile(fb200_plan* plan, const void* const* inputs, void* const* outputs,
                                 fb200_stream stream, float* step_ms, int cap, int* n_steps);
/* Op name of step `index` ("matmul+epilogue" when a following group was absorbed, "(absorbed)" /
 * "(alias)" for steps folded away).  The pointer is valid until the calling thread's next call. */
FB200_API const char* fb200_plan_step_op(const fb200_plan* plan, int index);

#ifdef __cplusplus
}
#endif
#endif /* FRAME_B200_H_ */
