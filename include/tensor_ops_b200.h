/*
 * tensor_ops_b200.h -- C ABI of the B200 (sm_100a) operator library.
 *
 * The first block re-declares, with identical names, argument order, struct layouts and enum
 * values, the entry points of the reference operator library that its Python operator classes
 * bind through ctypes (tensor_ops/tensor_ops.h in Sakauma/onnx_translator).  A process that
 * loads this library instead of the reference's tensor_ops.so gets the same functions; the one
 * difference is WHERE Tensor.data lives: it is a CUDA device pointer (or managed memory, see
 * tops_set_memory_mode), and every operator runs asynchronously on the library's stream.
 *
 * The second block (tops_*) is additive: transfers, streams, errors, zero-copy views and
 * fused operators that the reference has no counterpart for.
 *
 * There is no CPU fallback anywhere: without a usable CUDA device every call records an error
 * (tops_last_error) and create_tensor returns NULL.
 */
#ifndef TENSOR_OPS_B200_H
#define TENSOR_OPS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- types: tensor_ops/tensor_ops.h:10-54 ------------------------------------------------ */

/* tensor_ops/tensor_ops.h:10-23 (same numeric codes; Python mirrors them in nn/__init__.py:20-34) */
typedef enum {
    DTYPE_FLOAT8_E4M3 = 0,
    DTYPE_FLOAT8_E5M2 = 1,
    DTYPE_FLOAT16     = 2,
    DTYPE_BFLOAT16    = 3,
    DTYPE_FLOAT32     = 4,
    DTYPE_FLOAT64     = 5,
    DTYPE_INT4        = 6,   /* one value per byte, low nibble, sign-extended on read */
    DTYPE_INT8        = 7,
    DTYPE_UINT8       = 8,
    DTYPE_INT16       = 9,
    DTYPE_INT32       = 10,
    DTYPE_INT64       = 11
} DataType;

/* tensor_ops/tensor_ops.h:28-34.  Dense, row-major, no strides.  `data` is device memory;
   shape/ndim/size/dtype are host-readable. */
typedef struct {
    void*    data;
    int*     shape;
    int      ndim;
    size_t   size;
    DataType dtype;
} Tensor;

/* tensor_ops/tensor_ops.h:39-44.  Host arrays borrowed for the duration of the call.
   pads = [top, left, bottom, right] (only top and left are read, as in the reference),
   strides = [h, w], dilations = [h, w]. */
typedef struct {
    int* pads;
    int* strides;
    int* dilations;
    int  group;
} ConvParams;

/* tensor_ops/tensor_ops.h:49-54 */
typedef struct {
    int* pads;
    int* strides;
    int* dilations;
    int* kernel_shape;
} PoolParams;

/* ---- reference entry points ------------------------------------------------------------------ */

/* tensor_ops/tensor_ops.h:70 (tensor_ops.c:357-433).  Allocates from the current device's
   stream-ordered pool and zero-fills, like the reference's calloc.  NULL on failure. */
Tensor* create_tensor(int* shape, int ndim, DataType dtype);

/* tensor_ops/tensor_ops.h:77 (tensor_ops.c:440-450).  Drops one reference; the memory returns to
   the pool when the last reference (views included) is gone.  NULL is ignored. */
void free_tensor(Tensor* tensor);

/* tensor_ops/tensor_ops.h:91 (tensor_ops.c:763-807).  Builds the 4097-entry cosine table on the
   host and uploads it to the current device once.  cos_forward calls it on demand. */
void init_cos_lut(void);

/* tensor_ops/tensor_ops.h:85, 99, 107 (tensor_ops.c:708-757, 840-854).  input->size must equal
   output->size; otherwise nothing is computed, the output is zero-filled and an error recorded. */
void relu_forward(const Tensor* input, Tensor* output);
void cos_forward(const Tensor* input, Tensor* output);
void abs_forward(const Tensor* input, Tensor* output);

/* tensor_ops/tensor_ops.h:116-143 (tensor_ops.c:864-997).  The output dtype selects the
   arithmetic: integer outputs use saturating int64 arithmetic on round-to-nearest-even inputs,
   float64 outputs use double, other float outputs round the double result once more.
   Superset of the reference: an operand whose size differs from the output's is broadcast
   against the output shape (numpy rules, trailing dimensions aligned) instead of being rejected. */
void add_forward(const Tensor* A, const Tensor* B, Tensor* O);
void sub_forward(const Tensor* A, const Tensor* B, Tensor* O);
void mul_forward(const Tensor* A, const Tensor* B, Tensor* O);
void div_forward(const Tensor* A, const Tensor* B, Tensor* O);

/* tensor_ops/tensor_ops.h:149, 155 (tensor_ops.c:999-1034).
   Quantize:   y = saturate(rint(x / scale) + zero_point), scale == 0 -> zero_point; fp8 outputs
               encode that integer-valued result.
   Dequantize: y = (x - zero_point) * scale.
   Scale / ZeroPoint may be full-size (reference behaviour) or any shape that broadcasts against
   Y (e.g. [1], or [1,C,1,1] for per-axis). */
void quantize_linear_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint, Tensor* Y);
void dequantize_linear_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint, Tensor* Y);

/* tensor_ops/tensor_ops.h:161 (tensor_ops.c:1036-1114).  NCHW input, weights [M, C/group, KH, KW],
   optional bias [M] (NULL or NULL data = none), Y pre-shaped by the caller. */
void conv2d_forward(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, ConvParams* params);

/* tensor_ops/tensor_ops.h:166 (tensor_ops.c:1116-1165).  NCHW; padding taps are skipped. */
void max_pool_forward(const Tensor* X, Tensor* Y, PoolParams* params);

/* tensor_ops/tensor_ops.h:173 (tensor_ops.c:1167-1228).  Y = alpha * op(A) * op(B) + beta * C,
   C optional: scalar, 1-D of length N (per column) or M (per row), or >= 2-D with size-1
   broadcast on either of its last two dimensions. */
void gemm_forward(const Tensor* A, const Tensor* B, const Tensor* C, Tensor* Y,
                  float alpha, float beta, int transA, int transB);

/* tensor_ops/tensor_ops.h:179 (tensor_ops.c:1231-1270).  Softmax along `axis` (negative counts
   from the end). */
void softmax_forward(const Tensor* input, Tensor* output, int axis);

/* tensor_ops/tensor_ops.h:210, 216 (tensor_ops.c:1289-1299).  Byte copy between equal-size
   tensors (device to device). */
void flatten_forward(const Tensor* input, Tensor* output);
void reshape_forward(const Tensor* input, Tensor* output);

/* ---- operators around the hot path in exported CNNs (same signatures as the reference) -------- */

/* tensor_ops/tensor_ops.h:282 (tensor_ops.c:1497-1519).  Element-wise conversion.  float32 /
   float64 / float16 / bfloat16 sources going to an integer type are truncated toward zero, then
   saturated; every other pair is read as a double and stored like any operator result (so an fp8
   source going to an integer rounds to nearest-even). */
void cast_forward(const Tensor* input, Tensor* output);

/* tensor_ops/tensor_ops.h:276 (tensor_ops.c:1523-1543).  output = min(max(input, min), max) compared
   in double, lower bound first; either bound may be NULL; a NaN value or bound changes nothing.
   Superset: the bounds broadcast against the input (the reference wants them at full size). */
void clip_forward(const Tensor* input, Tensor* output, const Tensor* min, const Tensor* max);

/* tensor_ops/tensor_ops.h:464 (tensor_ops.c:2735-2789).  NCHW average pooling: double sum of the taps
   inside the plane in kh -> kw order divided by their number, or by the number of all taps when
   count_include_pad is set; a window without taps gives 0. */
void average_pool_forward(const Tensor* X, Tensor* Y, PoolParams* params, int count_include_pad);

/* tensor_ops/tensor_ops.h:466 (tensor_ops.c:2844-2868).  Mean of every H x W plane of a 4-D tensor
   (sequential double sum); output has one element per plane. */
void global_average_pool_forward(const Tensor* input, Tensor* output);

/* tensor_ops/tensor_ops.h:476 (tensor_ops.c:3041-3083).  Inference batch normalisation over dimension
   1: y = x * a + k with a = scale / sqrt(var + epsilon), k = B - mean * a, all in double, the product
   and the sum rounded separately. */
void batch_norm_forward(const Tensor* input, const Tensor* scale, const Tensor* B, const Tensor* mean,
                        const Tensor* var, Tensor* output, float epsilon);

/* tensor_ops/tensor_ops.h:230-240 (tensor_ops.c:1351-1403).  Element-wise maximum, minimum and power
   with the dtype dispatch and broadcasting of add_forward; pow_forward has no integer branch (pow() in
   double, then the store of the output type).  A NaN on either side of max / min yields B's element. */
void max_forward(const Tensor* A, const Tensor* B, Tensor* O);
void min_forward(const Tensor* A, const Tensor* B, Tensor* O);
void pow_forward(const Tensor* A, const Tensor* B, Tensor* O);

/* tensor_ops/tensor_ops.h:184-204, 265-298, 345-349, 441-452, 488-489, 507 (tensor_ops.c:595-604 and the
   one-line definitions at :1273-1286, :1484-1493, :1758-1760, :2622-2665, :3032-3035, :3340).  Element-wise
   functions: the element is read as a double, the expression is evaluated in double, the result is stored
   like any operator result.  neg, reciprocal, ceil, floor, sqrt, round, softsign and hard_swish are
   bit-identical to the reference; the transcendental ones agree to within one unit in the last place of a
   double before that store. */
void exp_forward(const Tensor* input, Tensor* output);
void log_forward(const Tensor* input, Tensor* output);
void sqrt_forward(const Tensor* input, Tensor* output);
void sigmoid_forward(const Tensor* input, Tensor* output);
void tanh_forward(const Tensor* input, Tensor* output);
void neg_forward(const Tensor* input, Tensor* output);
void reciprocal_forward(const Tensor* input, Tensor* output);
void ceil_forward(const Tensor* input, Tensor* output);
void floor_forward(const Tensor* input, Tensor* output);
void sin_forward(const Tensor* input, Tensor* output);
void tan_forward(const Tensor* input, Tensor* output);
void atan_forward(const Tensor* input, Tensor* output);
void softplus_forward(const Tensor* input, Tensor* output);
void softsign_forward(const Tensor* input, Tensor* output);
void hard_swish_forward(const Tensor* input, Tensor* output);
void acos_forward(const Tensor* input, Tensor* output);
void asin_forward(const Tensor* input, Tensor* output);
void cosh_forward(const Tensor* input, Tensor* output);
void sinh_forward(const Tensor* input, Tensor* output);
void asinh_forward(const Tensor* input, Tensor* output);
void acosh_forward(const Tensor* input, Tensor* output);
void atanh_forward(const Tensor* input, Tensor* output);
void round_forward(const Tensor* input, Tensor* output);
void erf_forward(const Tensor* input, Tensor* output);
void gelu_forward(const Tensor* input, Tensor* output);

/* tensor_ops/tensor_ops.h:298 (tensor_ops.c:1546-1606).  Y[..., m, n] = sum over k of A[..., m, k] * B[..., k, n];
   A, B and Y have rank >= 2 (the caller promotes 1-D operands), the leading dimensions broadcast numpy-style
   with operands of lower rank aligned to the right.  The sum runs in double in increasing k; 16-bit and 8-bit
   float operand pairs (and large float32 problems) use the tensor cores exactly as in gemm_forward. */
void matmul_forward(const Tensor* A, const Tensor* B, Tensor* Y);

/* tensor_ops/tensor_ops.h:547 (tensor_ops.c:3760-3809).  scale = (max(x, 0) - min(x, 0)) / 255 (1 if 0),
   zero point = round(-min / scale) clamped to 0..255, y = clamp(rint(x / scale) + zero point, 0, 255).
   y is uint8 in the reference's caller; any dtype is stored through the ordinary conversion.  y_scale and y_zp
   hold one element each. */
void dynamic_quantize_linear_forward(const Tensor* x, Tensor* y, Tensor* y_scale, Tensor* y_zp);

/* ---- additive interface (no counterpart in the reference) -------------------------------------- */

/* Error codes kept by the library (sticky until cleared; the first error wins). */
enum {
    TOPS_OK = 0,
    TOPS_ERR_INVALID = 1,      /* null tensor, size/shape mismatch, unsupported attribute */
    TOPS_ERR_CUDA = 2,         /* a CUDA runtime call failed (message holds its text)     */
    TOPS_ERR_NO_DEVICE = 3,    /* no usable CUDA device                                   */
    TOPS_ERR_OOM = 4,
    TOPS_ERR_UNSUPPORTED = 5,
    TOPS_ERR_DEVICE_TIMEOUT = 6 /* a bounded device-side wait expired                     */
};
int         tops_last_error(void);
const char* tops_last_error_message(void);
void        tops_clear_error(void);

/* Device and stream of the calling thread.  Default device: $TOPS_DEVICE, else $LOCAL_RANK,
   else 0.  Each device has one library-owned non-blocking stream; tops_set_stream substitutes
   a caller stream (cudaStream_t passed as void*), NULL restores the library's own. */
int   tops_set_device(int device);
int   tops_get_device(void);
int   tops_device_count(void);
void* tops_get_stream(void);
int   tops_set_stream(void* cuda_stream);
int   tops_sync(void);

/* 0 (default): cudaMallocAsync device memory.  1: CUDA managed memory plus a stream
   synchronise at the end of every operator, so that an unmodified host-side caller which
   memmove()s into Tensor.data and reads results back through the pointer keeps working. */
int tops_set_memory_mode(int managed);

/* A fixed sequence of operator calls as one CUDA graph (no counterpart in the reference, whose interpreter
   nn/__init__.py:408-456 walks the node list on every run).  Between tops_capture_begin and tops_capture_end the
   operator calls made on this thread's device are recorded instead of executed: kernels, memsets and the
   operators' own stream-ordered scratch.  Inside that window create no tensors, free none and transfer nothing:
   only operator calls on tensors that exist already and stay alive as long as the graph is used (same pointers
   on every launch).  tops_capture_launch enqueues the whole sequence on the current stream with one driver call.
   Not available in managed-memory mode.  tops_capture_end returns NULL (error recorded) when the sequence cannot
   be captured; the stream is usable again afterwards. */
int   tops_capture_begin(void);
void* tops_capture_end(void);
int   tops_capture_launch(void* captured);
void  tops_capture_free(void* captured);

/* Like create_tensor without the zero fill (operators overwrite the whole output). */
Tensor* tops_create_uninit(const int* shape, int ndim, DataType dtype);
/* Describe device memory owned by someone else (e.g. a framework tensor); never freed here. */
Tensor* tops_wrap(void* device_ptr, const int* shape, int ndim, DataType dtype);
/* Zero-copy reshape: a new Tensor header sharing base's memory and keeping it alive.
   The element count must match.  This is Flatten / Reshape without the copy. */
Tensor* tops_view(Tensor* base, const int* shape, int ndim);
/* Sub-range along dimension 0: rows [row_begin, row_begin + row_count) as a view (shards). */
Tensor* tops_slice_rows(Tensor* base, int row_begin, int row_count);
void    tops_retain(Tensor* tensor);

/* Host <-> device transfers on the current stream.  Upload returns after enqueueing when `host`
   is pinned (tops_host_alloc); download synchronises the stream before returning. */
int   tops_upload(Tensor* dst, const void* host, size_t nbytes);
int   tops_download(const Tensor* src, void* host, size_t nbytes);
int   tops_download_async(const Tensor* src, void* host, size_t nbytes);
void* tops_host_alloc(size_t nbytes);
void  tops_host_free(void* host);
size_t tops_dtype_size(DataType dtype);

/* Per-axis Q/DQ with 1-D scale / zero point of length shape[axis] (what the reference's Python
   class builds by reshaping, nn/Operators.py:439-445). */
void tops_quantize_linear_axis_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint,
                                       Tensor* Y, int axis);
void tops_dequantize_linear_axis_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint,
                                         Tensor* Y, int axis);

/* Quantize / Dequantize fused with their elementwise neighbours (no single counterpart in the reference: each call
   replaces a chain of its operators, tensor_ops.c:999-1034 with :864-997 add_forward and :708-728 relu_forward in
   between).  Results are bit-identical to the chain of separate calls.  Return TOPS_OK or the recorded error;
   TOPS_ERR_UNSUPPORTED (outputs zero-filled) means the caller runs the separate operators instead.

   tops_quantize_dequantize_forward:  Y = DequantizeLinear(QuantizeLinear(X, Scale, ZeroPoint), Scale, ZeroPoint)
     X, Scale, Y float32; Scale / ZeroPoint broadcast against X (one value, or [1,C,1,1] for per-axis); the code type
     is Codes->dtype (int8, uint8, float8) -- ZeroPoint has that type too, or int8 for float8 codes -- and, when
     Codes is NULL, ZeroPoint's type.  Codes, when given, receives what QuantizeLinear would store.
     Moves 8 bytes per element (9 with the codes) where the two operators move 10.

   tops_dq_add_q_forward:  Y = QuantizeLinear([Relu](DequantizeLinear(A, a_scale, a_zero) + DequantizeLinear(B, b_scale, b_zero)),
                                                y_scale, y_zero)
     A, B, Y int8 / uint8 codes of one element count; one float32 scale and one zero point of the tensor's own code
     type (NULL = 0) each.  Moves 3 bytes per element where the four or five operators move 27 or 35. */
int tops_quantize_dequantize_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint, Tensor* Codes, Tensor* Y);
int tops_dq_add_q_forward(const Tensor* A, const Tensor* a_scale, const Tensor* a_zero, const Tensor* B, const Tensor* b_scale,
                          const Tensor* b_zero, const Tensor* y_scale, const Tensor* y_zero, Tensor* Y, int relu);

/* Convolution for callers that must not let this library allocate GPU memory (no counterpart in
   the reference, whose library only ever uses the host heap).  conv2d_forward takes two scratch
   tensors from the CUDA memory pool on each call; a process that has given the whole device to its
   own allocator, runs under a fixed memory budget, or is in a phase where an allocation may block or
   fail cannot accept that.  This variant computes the same result with scratch in a fixed 36 MiB
   array inside the library image (held by every GPU on which the library's device code is loaded, until exit).
   Limits: the padded channels-last copy of X (N*Hp*Wp*C elements) must fit 32 MiB and the filter copy
   (KH*KW*M*C elements) 4 MiB; only what the tensor-core path covers is accepted (group 1, stride 1,
   fp16 / bf16 / fp8 inputs of one kind, fp32 / bf16 / fp16 output, C a multiple of 16 bytes).
   Anything else: output zero-filled, TOPS_ERR_UNSUPPORTED with the sizes in the message.
   The first call on a device resolves the array's device address (and creates the library stream
   if nothing ran there yet): make it before any stream capture.  All calls share the array, which
   keeps the previous call's contents (each call overwrites all it reads); calls that overlap on the
   GPU race, so keep them ordered on one stream.  tops_conv2d_noalloc_limits reports the limits.
   tops_conv2d_noalloc_prepare does the per-device set-up (stream, array address) ahead of time, outside
   the allocation-free phase, and creates the pinned host word through which an expired device-side wait
   is reported; without it (and without any earlier tensor-core operator call) such a time-out ends the
   kernel but is not reported.  Returns the error code. */
void   tops_conv2d_forward_noalloc(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, ConvParams* params);
int    tops_conv2d_noalloc_prepare(void);
size_t tops_conv2d_noalloc_limits(size_t* input_bytes, size_t* filter_bytes);

/* Fused forms of the operator sequences of quantised graphs (no single counterpart in the
   reference: each replaces a chain of its operators, nn/Operators.py:427-473 QuantizeLinear /
   DequantizeLinear followed by :613-669 Gemm or :475-548 Conv).  Scales are float32 tensors in
   device memory.  Return TOPS_OK or the recorded error; a case the tensor-core kernels do not
   cover is refused with TOPS_ERR_UNSUPPORTED (output zero-filled) and the caller runs the unfused
   chain instead.

   tops_gemm_qdq_forward:  Y = [QuantizeLinear]( alpha * DQ(A, a_scale) * DQ(B, b_scale)^T + beta * C )
     A, B fp8 codes (e4m3 / e5m2, zero point 0), one scale each; transA = 0, transB = 1.  With
     y_scale (one value) Y is an 8-bit type and receives rint(y / y_scale) stored the way
     quantize_linear_forward stores it; without it Y is float32 / bfloat16 / float16.

   tops_conv2d_dqw_forward:  Y = Conv(X, DQ(Wq, w_scale), B)
     Wq int8 codes with zero point 0 and one float32 scale per output channel; X float16 or
     bfloat16; group 1, stride 1. */
int tops_gemm_qdq_forward(const Tensor* A, const Tensor* a_scale, const Tensor* B, const Tensor* b_scale,
                          const Tensor* C, const Tensor* y_scale, Tensor* Y,
                          float alpha, float beta, int transA, int transB);
int tops_conv2d_dqw_forward(const Tensor* X, const Tensor* Wq, const Tensor* w_scale, const Tensor* B, Tensor* Y,
                            ConvParams* params);

/* The convolution of a QDQ network in one call, starting from the activation codes:
     Y = [Relu]( Conv( DQ(Xq, x_scale, x_zero), DQ(Wq, w_scale, 0) ) + B [+ R] )
   replaces DequantizeLinear (activations), DequantizeLinear (weights), Conv, an optional Add of a
   residual tensor R (float32, shape of Y, NULL for none) and an optional Relu
   (nn/Operators.py:452-473, 475-548, 170-200).  Xq int8 / uint8 NCHW with one scale and one zero
   point (x_zero may be NULL for 0), Wq int8 [M, C, KH, KW] with one float32 scale per output
   channel, B float32 or NULL, Y float32 / bfloat16 / float16.  Group 1; stride 1 with any dilation,
   or stride 2 with dilation 1; any C (the library pads channels in its scratch copy).  The integer
   levels are exact on the bfloat16 tensor path; see csrc/qconv.cu for the arithmetic. */
int tops_qlinear_conv_forward(const Tensor* Xq, const Tensor* x_scale, const Tensor* x_zero, const Tensor* Wq,
                              const Tensor* w_scale, const Tensor* B, const Tensor* R, Tensor* Y, ConvParams* params, int relu);

/* The same starting one operator earlier, from float32 activations:
     Y = [Relu]( Conv( DQ( Q(X, x_scale, x_zero), x_scale, x_zero ), DQ(Wq, w_scale, 0) ) + B [+ R] )
   replaces QuantizeLinear -> DequantizeLinear -> Conv [-> Relu] (nn/Operators.py:427-450 in addition
   to the operators named above).  The codes are those quantize_linear_forward would store, of the
   type of x_zero (int8 when x_zero is NULL). */
int tops_qdq_conv_forward(const Tensor* X, const Tensor* x_scale, const Tensor* x_zero, const Tensor* Wq,
                          const Tensor* w_scale, const Tensor* B, const Tensor* R, Tensor* Y, ConvParams* params, int relu);

/* The general form of the two calls above, which can also keep the activations between two
   quantised convolutions as integer levels: with y_levels the result is quantised with the NEXT
   convolution's input scale and zero point (the arithmetic of quantize_linear_forward) and stored
   as bfloat16 levels in the channels-last, zero-padded layout that convolution reads; passing that
   tensor as x with x_levels set skips the float32 tensor, the QuantizeLinear and the layout pass
   between the two.  The levels tensor has the shape tops_qconv_levels_shape reports for the
   convolution that will READ it and belongs to the caller; its padding cells and padding channels
   are never written, so it must be zero-filled (create_tensor) unless that shape equals [N, H, W, C].  y and y_levels may both be given. */
typedef struct QConvCall {
    const Tensor* x;            /* float32 NCHW values, int8 / uint8 NCHW codes, or (x_levels) bfloat16 levels */
    int x_levels;               /* non-zero: x was written as y_levels for this very convolution */
    int x_shape[4];             /* logical N, C, H, W of the input; read only when x_levels is set */
    const Tensor* x_scale;      /* float32[1] */
    const Tensor* x_zero;       /* int8 / uint8 [1] or NULL; ignored with x_levels (already subtracted) */
    const Tensor* w_codes;      /* int8 [M, C, KH, KW], zero point 0 */
    const Tensor* w_scale;      /* float32 [M] */
    const Tensor* bias;         /* float32 [M] or NULL */
    const Tensor* residual;     /* float32, the output's shape, or NULL */
    ConvParams* params;
    int relu;
    Tensor* y;                  /* float32 / bfloat16 / float16 NCHW, or NULL when only y_levels is wanted */
    Tensor* y_levels;           /* NULL, or bfloat16 levels for the next convolution */
    const Tensor* next_scale;   /* float32[1]: QuantizeLinear scale of the next convolution's input */
    const Tensor* next_zero;    /* its zero point (int8 / uint8 [1]) or NULL */
    ConvParams* next_params;    /* the next convolution's attributes ... */
    int next_kernel[2];         /* ... and filter extent KH, KW */
    Tensor** filter_cache;      /* NULL, or where the filters in the layout the tensor cores read are kept between calls:
                                   *filter_cache == NULL on the first call (the library creates and fills a tensor and
                                   stores it there), non-NULL afterwards (used as it is: same w_codes contents, same
                                   attributes, same kind of x).  The caller releases it with free_tensor. */
    /* Channels-last float32 edges.  The ABI's tensors are NCHW; a graph runner that owns the edge between two of
       these calls may keep it as [N, H, W, C] instead -- the order the tensor cores produce and consume -- and say
       so here.  Each flag describes one tensor of THIS call; the tensor's header carries the channels-last shape. */
    int x_channels_last;        /* x (float32 values or 8-bit codes, not levels) is [N, H, W, C] */
    int y_channels_last;        /* y is float32 [N, OH, OW, M] */
    int residual_channels_last; /* residual is float32 [N, OH, OW, M] */
} QConvCall;
int tops_qconv_forward(const QConvCall* call);
int tops_qconv_levels_shape(const int x_shape[4], const int kernel[2], const ConvParams* params, int levels_shape[4]);

/* The two halves of dynamic_quantize_linear_forward (tensor_ops.c:3760-3809), for a tensor whose rows are
   spread over several GPUs: each rank reduces its rows to range[0] = min, range[1] = max (float64[2] in
   device memory; NaNs never win, an empty tensor leaves +Inf / -Inf), the ranks combine their ranges
   (all-reduce with MIN / MAX), and each rank quantises its rows with the common range.  With one rank,
   range followed by apply equals dynamic_quantize_linear_forward bit for bit.  Return the error code. */
int tops_dynamic_quantize_range(const Tensor* x, Tensor* range);
int tops_dynamic_quantize_apply(const Tensor* x, const Tensor* range, Tensor* y, Tensor* y_scale, Tensor* y_zp);

/* Device-side exhaustive codec self-check: encodes every float32 bit pattern with the fast
   (hardware-convert) encoder and with the bit-level restatement of the reference encoder and
   returns the number of disagreements (NaN inputs excluded), or -1 on error. */
long long tops_selftest_encoder(DataType dtype);

/* Device-side exhaustive check of the fast table cosine: for every finite float32 input the
   reciprocal-multiply formulation must give the same double as the divide-based formulation of
   the reference.  Returns the number of disagreements, or -1 on error. */
long long tops_selftest_cos(void);

/* Device-side check of the bounded waits: one thread waits on a barrier that nothing arms, with a budget of
   `budget_microseconds` (1 .. 100000).  Returns 1 when the wait gave up as it must (0 if it claims to have succeeded,
   -1 on error); the expiry is also recorded like a real one, so the next tops_sync reports TOPS_ERR_DEVICE_TIMEOUT
   until tops_clear_error.  The kernel returns normally: nothing faults and the context stays usable. */
int tops_selftest_wait_timeout(int budget_microseconds);

/* Number of tensor-core (tcgen05) kernels launched so far by Gemm / Conv2d in this process: lets a
   caller tell that a call took the tensor-core path rather than the exact double-accumulating one. */
long long tops_tensor_core_launches(void);

/* Host-only (no CUDA call): the collapsed broadcast plan of one operand against an output shape:
   nd collapsed dimensions with their sizes and the operand's element strides (0 = broadcast);
   flat = 1 when the operand has the output's element count and is read at the output index.
   Returns 0 when the shapes do not broadcast.  Used by the CPU-side tests. */
int tops_debug_plan_broadcast(const int* out_shape, int out_ndim, const int* in_shape, int in_ndim,
                              int* nd, unsigned* sizes, int* strides, int* flat);

const char* tops_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TENSOR_OPS_B200_H */
