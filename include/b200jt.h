/*
 * b200jt.h -- C ABI of the B200 (sm_100a) kernels behind Jittor's meta-operator path.
 *
 * Conventions (all entry points):
 *   - plain C types only; tensors are described by b200jt_tensor (row-major, contiguous, <= 10 dims,
 *     like the reference's NanoVector shapes, python/jittor/src/misc/nano_vector.h:42-75);
 *   - the caller owns every buffer (inputs, outputs, workspace): nothing is allocated inside, which is
 *     the reference's rule too (the executor allocates all outputs before an op runs,
 *     python/jittor/src/executor.cc:575-577); the one exception is marked below;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call returns;
 *   - return value: 0 on success, <0 for an argument error, >0 for a CUDA error code;
 *     b200jt_last_error() gives the message of the calling thread's last failure;
 *   - device pointers must be valid on the current CUDA device.
 *
 * Paths in the comments are relative to the reference project root.
 */
#ifndef B200JT_H_
#define B200JT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200JT_MAX_DIMS 10
#define B200JT_MAX_EXTRAS 10

/* dtype codes (the reference's dtype names, python/jittor/src/misc/nano_string.h) */
enum b200jt_dtype {
    B200JT_BOOL = 0, B200JT_INT8 = 1, B200JT_INT16 = 2, B200JT_INT32 = 3, B200JT_INT64 = 4,
    B200JT_UINT8 = 5, B200JT_FLOAT16 = 6, B200JT_BFLOAT16 = 7, B200JT_FLOAT32 = 8, B200JT_FLOAT64 = 9
};

typedef struct b200jt_tensor {
    void*   ptr;                       /* device pointer (may be NULL iff the tensor has 0 elements) */
    int32_t dtype;                     /* enum b200jt_dtype */
    int32_t ndim;                      /* 1..B200JT_MAX_DIMS */
    int64_t shape[B200JT_MAX_DIMS];
} b200jt_tensor;

const char* b200jt_last_error(void);
int         b200jt_version(void);

/* Classifies index strings: returns 1 and fills coef[d*B200JT_MAX_DIMS + j], c0[d] if every index d is
 * c0[d] + sum_j coef[d][j]*i_j (no @e loads), 0 if not affine, <0 on a syntax error. This is what the
 * reference's tuners recover with expr::match on the same strings (python/jittor/src/opt/tuner/conv_tuner.cc:313-338). */
int b200jt_index_affine(const int64_t* loop_shape, int ndim_loop, const int64_t* x_shape, int ndim_x,
                        const char* const* indexes, int n_indexes, int64_t* coef, int64_t* c0);

/* ---- meta-operators --------------------------------------------------------------------------- */

/* y[i] = overflow(i) ? overflow_value : x[index_0(i), ..., index_m(i)].
 * Replaces ReindexOp(Var* x, NanoVector shape, vector<string>&& indexes, float64 overflow_value,
 *                    vector<string>&& overflow_conditions, vector<Var*>&& extras)
 * python/jittor/src/ops/reindex_op.h:91 and its jit_run, python/jittor/src/ops/reindex_op.cc:111-139.
 * `indexes` are C integer expressions over i0..in, shape symbols and @eK(...) loads of extras. */
int b200jt_reindex(const b200jt_tensor* x, const b200jt_tensor* y,
                   const char* const* indexes, int n_indexes, double overflow_value,
                   const char* const* overflow_conditions, int n_conditions,
                   const b200jt_tensor* extras, int n_extras, void* stream);

/* The CUDA source the library compiles for this reindex once it has seen the same op instance twice (affine index
 * expressions, every tensor below 2^31 elements, at least 2^16 outputs; B200JT_REINDEX_JIT=0 switches the run-time
 * specialisation off, =2 compiles at first sight and makes a failure an error). Nothing is launched and the pointers are
 * only looked at for their alignment, so no GPU is needed. Copies at most cap bytes, NUL-terminated, into src (may be
 * NULL), stores the full length in *needed (0 when the op is not of the compiled kind) and sets *compiled to 1 if NVRTC
 * accepted the source for sm_100a. Counterpart of reading the reference's generated reindex source
 * (python/jittor/src/ops/reindex_op.cc:93-109 fills the index expressions into the loop nest it compiles). */
int b200jt_reindex_source(const b200jt_tensor* x, const b200jt_tensor* y, const char* const* indexes, int n_indexes,
                          double overflow_value, const char* const* overflow_conditions, int n_conditions,
                          const b200jt_tensor* extras, int n_extras, char* src, int64_t cap, int64_t* needed, int* compiled);

/* x[:] = init(op); for every i of y: if !overflow(i): x[index(i)] = op(x[index(i)], y[i]).
 * Replaces ReindexReduceOp(Var* y, NanoString op, NanoVector shape, vector<string>&& indexes,
 *                          vector<string>&& overflow_conditions, vector<Var*>&& extras)
 * python/jittor/src/ops/reindex_reduce_op.h:86, jit_run python/jittor/src/ops/reindex_reduce_op.cc:93-131.
 * op: add multiply maximum minimum bitwise_and bitwise_or bitwise_xor logical_and logical_or logical_xor void.
 * `workspace` must hold b200jt_reindex_reduce_workspace(...) bytes (may be 0). */
size_t b200jt_reindex_reduce_workspace(const b200jt_tensor* y, const b200jt_tensor* x, const char* op,
                                       const char* const* indexes, int n_indexes,
                                       const char* const* overflow_conditions, int n_conditions,
                                       const b200jt_tensor* extras, int n_extras);
int b200jt_reindex_reduce(const b200jt_tensor* y, const b200jt_tensor* x, const char* op,
                          const char* const* indexes, int n_indexes,
                          const char* const* overflow_conditions, int n_conditions,
                          const b200jt_tensor* extras, int n_extras,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Same operation as b200jt_reindex_reduce for callers that may not allocate device memory when they call
 * (inside an allocator callback, in a loop whose memory pool is frozen after start-up, behind a plugin
 * interface without an allocation hook). It has no counterpart in the reference. The scratch rows the
 * few-bins scatter needs are kept in a 4 MiB array that is part of the library image on every GPU that loads
 * it; b200jt_reindex_reduce_noalloc_max_scratch() returns that size. A scatter whose plan needs more
 * (float32 bins beyond about 7000) is refused with status -3 and a message naming both sizes; nothing is
 * allocated or freed on any path. The first call on a device looks up the array's device address, so make
 * that call before any stream capture. All calls share the one array and its contents persist between calls
 * (every launch overwrites all rows it reads, nothing needs zeroing), therefore two calls that may overlap on
 * the GPU -- different streams, or threads -- race and must be serialised by the caller. */
size_t b200jt_reindex_reduce_noalloc_max_scratch(void);
int b200jt_reindex_reduce_noalloc(const b200jt_tensor* y, const b200jt_tensor* x, const char* op,
                                  const char* const* indexes, int n_indexes,
                                  const char* const* overflow_conditions, int n_conditions,
                                  const b200jt_tensor* extras, int n_extras, void* stream);

/* out = x; for every element i of data: out[index_0(i), ...] = op(out[...], data[i]); op "void" assigns.
 * Replaces SetitemOp(Var* x, VarSlices&& slices, Var* y, NanoString op), python/jittor/src/ops/setitem_op.h:24, jit_run
 * python/jittor/src/ops/setitem_op.cc:268-366: the host turns the slices into one index expression per axis of x
 * (loop variable, start + step * loop variable, constant, formula string, or @eK load of an index Var) and broadcasts
 * data to the shape of the sliced region. x and out may be the same buffer (the reference's in-place form).
 * op: void add multiply maximum minimum bitwise_and/or/xor logical_and/or/xor. */
int b200jt_setitem(const b200jt_tensor* x, const b200jt_tensor* data, const b200jt_tensor* out, const char* op,
                   const char* const* indexes, int n_indexes,
                   const b200jt_tensor* extras, int n_extras, void* stream);

/* z[i] = x[i with the axes of bcast_mask zeroed]; x is passed with z's rank (size-1 axes where broadcast).
 * Replaces BroadcastToOp(Var* x, NanoVector shape, uint dims_mask, uint keepdims_mask)
 * python/jittor/src/ops/broadcast_to_op.h:90, jit_run python/jittor/src/ops/broadcast_to_op.cc:177-194. */
int b200jt_broadcast_to(const b200jt_tensor* x, const b200jt_tensor* z, uint32_t bcast_mask, void* stream);

/* y = reduce_op over the axes of reduce_mask (y passed with x's rank, size-1 on reduced axes).
 * Replaces ReduceOp(Var* x, NanoString op, uint dims_mask, uint keepdims_mask)
 * python/jittor/src/ops/reduce_op.h:19, jit_run python/jittor/src/ops/reduce_op.cc:374-399.
 * op: add mean multiply maximum minimum bitwise_and/or/xor logical_and/or/xor. */
size_t b200jt_reduce_workspace(const b200jt_tensor* x, const b200jt_tensor* y, const char* op, uint32_t reduce_mask);
int b200jt_reduce(const b200jt_tensor* x, const b200jt_tensor* y, const char* op, uint32_t reduce_mask,
                  void* workspace, size_t workspace_bytes, void* stream);

/* ---- element-wise ops fused around them ------------------------------------------------------- */

/* z = op(x, y); x and y may have size-1 axes where z does not (the broadcast_to the reference inserts,
 * python/jittor/src/ops/binary_op.cc:435-441, fused into the same kernel). All three have z's rank.
 * Replaces BinaryOp(Var* x, Var* y, NanoString op), python/jittor/src/ops/binary_op.h:14, jit_run
 * python/jittor/src/ops/binary_op.cc:563-570; scalar semantics python/jittor/src/type/common_op_type.cc:82-152. */
int b200jt_binary(const b200jt_tensor* x, const b200jt_tensor* y, const b200jt_tensor* z, const char* op, void* stream);

/* y = op(x); a dtype name as op is a cast. Replaces UnaryOp(Var* x, NanoString op), python/jittor/src/ops/unary_op.h:16. */
int b200jt_unary(const b200jt_tensor* x, const b200jt_tensor* y, const char* op, void* stream);

/* z = cond ? x : y. Replaces TernaryOp(Var* cond, Var* x, Var* y), python/jittor/src/ops/ternary_op.h:14. */
int b200jt_ternary(const b200jt_tensor* cond, const b200jt_tensor* x, const b200jt_tensor* y,
                   const b200jt_tensor* z, void* stream);

/* ---- fused chains (what op_compiler/FusedOp + the tuners produce for the nn callers) ----------- */

/* Any chain of unary / binary / ternary ops, broadcasts and reduces over the trailing axes as ONE launch, intermediates
 * in registers: the general case of FusedOp::jit_run -- the loop nest OpCompiler stitches from the member ops
 * (python/jittor/src/fused_op.cc:41-118,217-238, python/jittor/src/op_compiler.cc:839-1045; fused reduce + broadcast
 * cases python/jittor/test/test_fused_op.py:144-176). The reference generates and compiles a loop nest per graph; here
 * the graph is passed as a small program, and the kernel that runs it is specialised for that program at first use
 * (straight-line CUDA generated from the program, compiled for sm_100a with NVRTC, cached per process; constants, shapes,
 * strides and pointers stay arguments, so one compilation serves every size; the cubins are also kept on disk under
 * $B200JT_CACHE_DIR, default ~/.cache/b200jt, "0" = off, so a later process loads instead of compiling). Without NVRTC, or with
 * B200JT_CHAIN_JIT=0, an ahead-of-time kernel interprets the program instead (same results, slower);
 * B200JT_CHAIN_JIT=2 makes a missing compiler or a failed compilation an error.
 *   inputs      n_inputs (<= 8) tensors, each with the rank of full_shape, size 1 on the axes it is broadcast over;
 *   full_shape  the index space of the element-wise part; its last row_axes axes form a "row" (the axes the program's
 *               reduces fold; 0 when there is no reduce);
 *   code        32-bit words  op | sub << 4 | kind << 10 | index << 13 | swap << 21 | result_dtype << 24  for an
 *               accumulator machine (result_dtype: enum b200jt_dtype of the node, float32 / bfloat16 / float16 / bool;
 *               every op computes in float32 and rounds to it). An operand is (kind, index): 1 input k, 2 constant (the
 *               float32 in the next word), 3 row value j, 4 temporary t (t < 6).
 *                 1 LOAD o         acc = o                       2 UNARY (sub = u)     acc = u(acc)
 *                 3 BINARY (sub = b) o   acc = acc b o, or o b acc if swap
 *                 4 SELECT o1, then a word with op 0 holding o2      acc = acc != 0 ? o1 : o2
 *                 5 TSTORE t       tmp[t] = acc
 *               statements end a chain:
 *                 8 ROW_REDUCE (sub = reduce_op, index = j)  rowval[j] = fold of acc over the row (add, mean, maximum, minimum, multiply)
 *                 9 ROW_MAP j      rowval[j] = acc (a chain of row values, per-row inputs, constants)
 *                10 STORE          out = acc (full_shape; must be last)       11 STORE_ROW j   out[row] = rowval[j] (last)
 *               u: index in {cast, negative, abs, logical_not, bitwise_not, log, exp, sqrt, round, floor, ceil, sin, asin,
 *               sinh, asinh, tan, atan, tanh, atanh, cos, acos, cosh, acosh, sigmoid, erf, erfinv}; b / reduce_op: index in
 *               {add, subtract, multiply, divide, floor_divide, mod, pow, maximum, minimum, less, less_equal, greater,
 *               greater_equal, equal, not_equal, logical_and, logical_or, logical_xor} and 23 = mean;
 *   out         full_shape elements (STORE) or one per row (STORE_ROW). */
int b200jt_fused_chain(const b200jt_tensor* inputs, int n_inputs, const int64_t* full_shape, int ndim, int row_axes,
                       const int32_t* code, int n_code, const b200jt_tensor* out, void* stream);

/* The CUDA source b200jt_fused_chain would compile for the same arguments, without launching anything (the pointers in
 * the descriptors are only looked at for their alignment; needs no GPU). Copies at most cap bytes, NUL-terminated, into
 * src (may be NULL), stores the full length in *needed and sets *compiled to 1 if NVRTC accepted the source for sm_100a
 * (0, with the compiler's log in b200jt_last_error(), otherwise). The counterpart of reading the reference's generated
 * op source under its cache directory (python/jittor/src/op_compiler.cc:1046-1060 writes it). */
int b200jt_fused_chain_source(const b200jt_tensor* inputs, int n_inputs, const int64_t* full_shape, int ndim, int row_axes,
                              const int32_t* code, int n_code, const b200jt_tensor* out, char* src, int64_t cap,
                              int64_t* needed, int* compiled);

/* Counters of the chain specialiser since the process started: kernels compiled, launches served from the cache,
 * compilations that failed (those chains run through the interpreting kernel). Any pointer may be NULL.
 * No reference counterpart (the reference logs its compilations through LOGvv). */
int b200jt_chain_jit_stats(int* compiled, int* hits, int* failed);

/* Row softmax / log-softmax over the last axis of x[rows, cols], one read and one write.
 * Replaces the chain of python/jittor/nn.py:527-535 and the inline kernel python/jittor/other/code_softmax.py:42-98.
 * x, y: float32 or bfloat16 (fp32 math). */
int b200jt_softmax(const b200jt_tensor* x, const b200jt_tensor* y, int log, void* stream);

/* Gradient of the above over the last axis from the forward OUTPUT y and the output gradient dy:
 * dx = y * (dy - sum(y*dy)) (softmax) or dy - exp(y) * sum(dy) (log-softmax), one read of y and dy, one write.
 * Replaces the backward kernel of python/jittor/other/code_softmax.py:109-147. y, dy, dx: float32 or bfloat16, same dtype. */
int b200jt_softmax_backward(const b200jt_tensor* y, const b200jt_tensor* dy, const b200jt_tensor* dx, int log, void* stream);

/* Row LayerNorm over the last axis: mean, E[x^2], var = max(E[x^2]-E[x]^2, 0), y = x*w + b with
 * w = gamma/sqrt(var+eps), b = beta - mean*w. gamma/beta may be NULL (1 and 0).
 * Replaces the chain of python/jittor/nn.py:778-787. x, y: float32 or bfloat16; gamma, beta: float32 [cols]. */
int b200jt_layer_norm(const b200jt_tensor* x, const b200jt_tensor* gamma, const b200jt_tensor* beta,
                      const b200jt_tensor* y, double eps, void* stream);

/* c = op_a(a) . op_b(b), fp32 accumulation. Replaces the relay
 * CublasMatmulOp(Var* a, Var* b, bool trans_a, bool trans_b), python/jittor/extern/cuda/cublas/ops/cublas_matmul_op.h:18,
 * chosen by MatmulTuner for reduce.add(multiply(broadcast_to(a), broadcast_to(b))), python/jittor/src/opt/tuner/matmul_tuner.cc:21-102.
 * a, b, c: float32 or bfloat16, same dtype. */
size_t b200jt_matmul_workspace(const b200jt_tensor* a, const b200jt_tensor* b, const b200jt_tensor* c, int trans_a, int trans_b);
int b200jt_matmul(const b200jt_tensor* a, const b200jt_tensor* b, const b200jt_tensor* c,
                  int trans_a, int trans_b, void* workspace, size_t workspace_bytes, void* stream);

/* c[i] = op_a(a[i]) . op_b(b[i]), i < batch, in one launch: a [Ba, ., .], b [Bb, ., .], c [batch, M, N], Ba and Bb equal to
 * batch or 1 (an operand with batch extent 1 is shared by all products). Replaces the relay
 * CublasBatchedMatmulOp(Var* a, Var* b, bool trans_a, bool trans_b), python/jittor/extern/cuda/cublas/ops/cublas_batched_matmul_op.h:21,
 * jit_run python/jittor/extern/cuda/cublas/ops/cublas_batched_matmul_op.cc:100-175 (cublasGemmStridedBatchedEx), which
 * nn.matmul / nn.bmm call for [..., n, m] x [..., m, k] (python/jittor/nn.py:127-131). float32 or bfloat16, fp32 accumulation. */
int b200jt_batched_matmul(const b200jt_tensor* a, const b200jt_tensor* b, const b200jt_tensor* c,
                          int trans_a, int trans_b, void* stream);

/* Status word of the kernels that wait (matmul, conv2d, peer all-reduce): every wait inside them is bounded; if
 * one expires the kernel stops cleanly and records which (1 producer, 2 accumulator hand-back, 3 operand arrival,
 * 4 accumulator ready, 5 a peer's flag in b200jt_peer_all_reduce). Returns 0 if none did since the last call, and clears the word. Synchronises the device. It plays the
 * role of the reference's checkCudaErrors after a relay (python/jittor/extern/cuda/cublas/ops/cublas_matmul_op.cc:117). */
int b200jt_device_status(void);

/* y = conv2d(x, w), NCHW ("abcd") x, OIHW w, fp32 accumulation. Replaces the relay
 * CudnnConvOp(Var* x, Var* w, int strideh, int stridew, int paddingh, int paddingw, int dilationh, int dilationw,
 *             int groups, string xformat, string wformat, string yformat),
 * python/jittor/extern/cuda/cudnn/ops/cudnn_conv_op.h:17, chosen by ConvTuner for
 * reduce.add(multiply(reindex(x), broadcast_to(w))), python/jittor/src/opt/tuner/conv_tuner.cc:218-411.
 * groups > 1: w is [Cout, Cin/groups, KH, KW] (python/jittor/nn.py:1022-1056); grouped shapes run on the CUDA-core kernel.
 * If stats != NULL (float32 [2*Cout], zeroed by the callee) it also receives per-channel sum(y) and sum(y*y):
 * the reduce of python/jittor/nn.py:674-675 fused into the conv epilogue. */
size_t b200jt_conv2d_workspace(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                               int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int groups);
int b200jt_conv2d(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                  int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int groups,
                  float* stats, void* workspace, size_t workspace_bytes, void* stream);

/* The same convolution with the layout strings of the reference's relay (CudnnConvOp(..., string xformat, string wformat,
 * string yformat), python/jittor/extern/cuda/cudnn/ops/cudnn_conv_op.h; ConvTuner derives them,
 * python/jittor/src/opt/tuner/conv_tuner.cc:292-341): xformat / yformat "abcd" (NCHW) or "acdb" (NHWC, shape given as
 * [N, H, W, C]), wformat "oihw" or "ohwi" ([Cout, KH, KW, Cin]); an empty yformat follows xformat. groups == 1.
 * Layouts other than abcd / oihw run on the tensor-core kernel only (bfloat16, in channels a multiple of 8 and >= 64, out
 * channels >= 64): NHWC is that kernel's native operand layout, so an acdb input skips the layout pass and an acdb output is
 * written by the epilogue directly -- a conv -> conv chain kept in acdb pays no layout pass at all. */
size_t b200jt_conv2d_formats_workspace(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                                       int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                                       const char* xformat, const char* wformat, const char* yformat);
int b200jt_conv2d_formats(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                          int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                          const char* xformat, const char* wformat, const char* yformat,
                          float* stats, void* workspace, size_t workspace_bytes, void* stream);

/* y = conv_transpose2d(x, w): y[n,o,ho,wo] = sum x[n,i,hi,wi] * w[i,o,kh,kw] over ho = hi*stride - pad + kh*dil (same for w),
 * x NCHW, w [Cin, Cout/groups, KH, KW], fp32 accumulation. y's spatial shape carries the output_padding. Replaces the
 * relay CudnnConvBackwardXOp(Var* w, Var* y, int height, int width, int strideh, ..., int groups, ...),
 * python/jittor/extern/cuda/cudnn/ops/cudnn_conv_backward_x_op.h:20, which ConvTuner selects for
 * reindex_reduce.add(multiply(broadcast(x), broadcast(w))), python/jittor/src/opt/tuner/conv_tuner.cc:375-397 -- the graph
 * ConvTranspose.execute builds (python/jittor/nn.py:1429-1491). */
int b200jt_conv2d_transpose(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                            int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int groups, void* stream);

/* dw[o,c,kh,kw] = sum over (n,oh,ow) of dy[n,o,oh,ow] * x[n,c,oh*stride-pad+kh*dil, ...]: the weight gradient of conv2d
 * (groups == 1), fp32 accumulation. Replaces the relay CudnnConvBackwardWOp(Var* x, Var* y, int kh, int kw, int strideh, ...),
 * python/jittor/extern/cuda/cudnn/ops/cudnn_conv_backward_w_op.h:20, which ConvTuner selects for
 * reduce.add(multiply(reindex(x), broadcast(dy))), python/jittor/src/opt/tuner/conv_tuner.cc:375-397. */
int b200jt_conv2d_backward_w(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                             int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, void* stream);

/* The same weight gradient with a workspace: bfloat16 layers (in and out channels multiples of 8 and >= 64, strides <= 4,
 * output at least 8 x 8 per image and 4096 pixels in all, 16-byte aligned x and dy) run on the tensor cores -- x and dy
 * are copied to channels-last form, each CTA accumulates one (tap, 128 in channels, 256 out channels) block over a range
 * of pixels in fp32, and the ranges are added in a fixed order, so results repeat bit for bit. The _workspace query
 * returns the bytes that path needs (0: it does not apply; the call then runs the kernel of b200jt_conv2d_backward_w and
 * takes no workspace). Replaces the same relay, cudnnConvolutionBackwardFilter with its workspace,
 * python/jittor/extern/cuda/cudnn/ops/cudnn_conv_backward_w_op.cc:292. */
size_t b200jt_conv2d_backward_w_workspace(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                                          int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w);
int b200jt_conv2d_backward_w_tc(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                                int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                                void* workspace, size_t workspace_bytes, void* stream);

/* The weight gradient with the relay's layout strings (CudnnConvBackwardWOp(..., string xformat, string wformat, string
 * yformat), python/jittor/extern/cuda/cudnn/ops/cudnn_conv_backward_w_op.h:20; layouts as ConvTuner derives them,
 * python/jittor/src/opt/tuner/conv_tuner.cc:292-341): xformat describes x and yformat dy, "abcd" (NCHW) or "acdb" (NHWC, read
 * by the kernel as they are: no copy on that side); wformat describes dw, "oihw" or "ohwi". Layouts other than
 * abcd / oihw / abcd exist on the tensor-core kernel only (status -5 where it does not apply). */
size_t b200jt_conv2d_backward_w_formats_workspace(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                                                  int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                                                  const char* xformat, const char* wformat, const char* yformat);
int b200jt_conv2d_backward_w_formats(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                                     int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                                     const char* xformat, const char* wformat, const char* yformat,
                                     void* workspace, size_t workspace_bytes, void* stream);

/* Per-channel sum(x) and sum(x*x) of x[N,C,H,W] into stats[2*C] (float32): the two reduce.mean of
 * BatchNorm.execute, python/jittor/nn.py:674-675, in one pass, unnormalised so that ranks can be
 * summed by an all-reduce (python/jittor/nn.py:676-678). */
int b200jt_bn_stats(const b200jt_tensor* x, float* stats, void* stream);

/* y = [relu](x*w + b), w = gamma/sqrt(var+eps), b = beta - mean*w with mean = stats[c]/count,
 * var = max(stats[C+c]/count - mean^2, 0): python/jittor/nn.py:680-683 (+ nn.relu). If running_mean / running_var
 * (float32 [C], both or neither) are given they are updated in place, running += (batch - running) * momentum, the
 * two Var.update calls of python/jittor/nn.py:684-688. */
int b200jt_bn_apply(const b200jt_tensor* x, const float* stats, double count, const float* gamma, const float* beta,
                    double eps, int relu, const b200jt_tensor* y,
                    float* running_mean, float* running_var, double momentum, void* stream);

/* ---- pooling ----------------------------------------------------------------------------------------
 * y[n,c,oh,ow] = op over the window rows [oh*sh-ph, +kh) x columns [ow*sw-pw, +kw) of x[n,c], clipped to x. Replaces the
 * jt.code kernels of Pool.execute, python/jittor/pool.py:42-197 (forward body :54-81, backward body :82-95):
 * op "maximum" / "minimum" start from the op's init value; "mean" divides by kh*kw when count_include_pad, else by the
 * clipped window area. y's spatial shape selects floor or ceil mode (python/jittor/pool.py:46-53). indices (maximum /
 * minimum, may be NULL) receives p*W+q of the first extreme element, -1 for an empty window (:70-81).
 * Backward: dx[n,c,p,q] = sum of dy over the windows in which x[n,c,p,q] is the FIRST element (row-major) equal to
 * y (maximum / minimum), or sum of dy/count over the windows containing it (mean). dtypes: float32/64, float16, bfloat16. */
int b200jt_pool2d(const b200jt_tensor* x, const b200jt_tensor* y, int32_t* indices, const char* op,
                  int kh, int kw, int sh, int sw, int ph, int pw, int count_include_pad, void* stream);
int b200jt_pool2d_backward(const b200jt_tensor* x, const b200jt_tensor* y, const b200jt_tensor* dy, const b200jt_tensor* dx,
                           const char* op, int kh, int kw, int sh, int sw, int ph, int pw, int count_include_pad, void* stream);
/* The same gradient for maximum / minimum from the index map the forward produced (x and y only give the geometry, they
 * are not read): element (p, q) receives dy of every window whose index is p*W+q. Identical results, less traffic. */
int b200jt_pool2d_backward_indices(const b200jt_tensor* x, const b200jt_tensor* y, const int32_t* indices,
                                   const b200jt_tensor* dy, const b200jt_tensor* dx,
                                   int kh, int kw, int sh, int sw, int ph, int pw, void* stream);

/* ---- all-reduce over NVLink peer mappings --------------------------------------------------------
 * y = op over the ranks of x, one kernel per rank that reads and writes the other ranks' memory directly: replaces
 * the relay NcclAllReduceOp(Var* x), python/jittor/extern/cuda/nccl/ops/nccl_all_reduce_op.h:14, jit_run
 * python/jittor/extern/cuda/nccl/ops/nccl_all_reduce_op.cc:46-58 (ncclAllReduce(xp, yp, y->num, T, ncclSum, comm, 0)),
 * which MpiAllReduceOp forwards to on CUDA (python/jittor/extern/mpi/ops/mpi_all_reduce_op.cc:39-47). The reference
 * sums only; "maximum" and "minimum" are accepted too (what a scatter-max onto a shared output needs).
 * Set-up, once per process: every rank creates a segment (device memory holding flags and four staging areas of
 * data_bytes each; the IPC handle is what the other ranks open), the 64-byte handles are exchanged by the host
 * (rank order), and b200jt_peer_comm_create maps them. A call reduces count elements of dtype (float32/64, int32/64,
 * float16/bfloat16 with float32 accumulation) from src into dst (may alias), count*size <= data_bytes; all ranks
 * must issue the same sequence of calls. Sums run in rank order on every rank: all ranks receive identical bits.
 * Only kernel launches are issued, so calls can be captured in a CUDA graph. A peer that does not arrive within
 * wait_ms makes the kernel return with status 5 (b200jt_device_status); the communicator must then be rebuilt. */
#define B200JT_IPC_HANDLE_BYTES 64
#define B200JT_PEER_MAX_RANKS 8
size_t b200jt_peer_segment_bytes(size_t data_bytes);
int b200jt_peer_segment_create(size_t data_bytes, void** segment, unsigned char* ipc_handle);
int b200jt_peer_segment_destroy(void* segment);   /* only for a segment no communicator took over (set-up failed elsewhere) */
int b200jt_peer_comm_create(int rank, int world, void* own_segment, const unsigned char* ipc_handles,
                            size_t data_bytes, double wait_ms, void** comm);
int b200jt_peer_comm_destroy(void* comm);
size_t b200jt_peer_max_bytes(const void* comm);
/* Running the collective BESIDE the next kernel instead of between two kernels (the reference serialises both on stream 0,
 * python/jittor/extern/cuda/nccl/ops/nccl_all_reduce_op.cc:57): b200jt_peer_comm_set_max_blocks caps the CTAs of one
 * all-reduce call (0 = no cap; every rank must use the same value), and b200jt_set_sm_reserve(sms) makes the persistent
 * kernels of this library size their grids for 148 - sms SMs, so that the collective's CTAs find room while they run. */
int b200jt_peer_comm_set_max_blocks(void* comm, int max_blocks);
int b200jt_set_sm_reserve(int sms);
int b200jt_peer_all_reduce(void* comm, const void* src, void* dst, int64_t count, int dtype, const char* op, void* stream);
/* The same job with all ranks on ONE device (test aid and single-GPU emulation): `world` communicators whose segments
 * live side by side, and one cooperative launch that plays every rank (blocks wait on one another, so they have
 * to be co-resident; messages are limited accordingly by the launch failing, never by a hang). */
int b200jt_peer_comm_create_local(int world, size_t data_bytes, double wait_ms, void** comms);
int b200jt_peer_all_reduce_local(void* const* comms, int world, const void* const* srcs, void* const* dsts,
                                 int64_t count, int dtype, const char* op, void* stream);

/* ---- diagnostics ---------------------------------------------------------------------------------
 * Operation rates (1e9 per second) of the atomic units the scatter kernels lean on, each measured with one small kernel:
 * "red_global" (red.global.add.u32 to random words of a `words`-word table: the ceiling of a one-atomic-per-element
 * scatter), "smem_int", "smem_float" (shared-memory atomicAdd on 4096 words), "match_any". skewed != 0 sends about 16 % of
 * the shared-memory operations to one address. Synchronises the device; scratch holds max(words * 4, 1024) bytes.
 * The reference's profiler reports achieved bandwidth per kernel (python/jittor/src/profiler/profiler.cc:148-183); it has no
 * counterpart of this probe. */
int b200jt_probe_rate(const char* what, int skewed, void* scratch, int64_t words, double* gops);

#ifdef __cplusplus
}
#endif
#endif /* B200JT_H_ */
