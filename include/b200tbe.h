/*
 * b200tbe.h -- C ABI of libb200tbe.so: table-batched embedding (TBE) lookups, the TBE backward
 * with a fused row-wise optimizer, and the jagged-tensor copies, as CUDA kernels for sm_100a.
 *
 * Every entry point takes a POD parameter block of raw DEVICE pointers plus a CUDA stream, enqueues
 * its kernels on that stream and returns without synchronising. The return value is B200TBE_OK or
 * a negative b200tbe_status. Nothing here allocates device memory except where a function says so:
 * scratch is passed in by the caller, sized by the matching *_scratch_bytes() query.
 *
 * The intel/torchlib-xpu tree that this library plugs into has no FBGEMM plugin of its own; its one
 * plugin shows the pattern this boundary replaces: a host library registered at load time
 * (packages/torchcodec-xpu/src/torchcodec_xpu/XpuDeviceInterface.cpp:33-35) which fetches the
 * caller's current stream (XpuDeviceInterface.cpp:415) and hands raw pointers and sizes to a free
 * function that launches the device kernel
 * (packages/torchcodec-xpu/src/torchcodec_xpu/ColorConversionKernel.h:12-20). Each entry point
 * below names the torch.ops.fbgemm operator whose device half it is; the tensor conventions are
 * those of FBGEMM's embedding kernels (include/fbgemm/FbgemmEmbedding.h:26-38 for the pooling
 * semantics, :58-62 for offsets, :90-93 and :147-150 for the quantised row layout).
 */
#ifndef B200TBE_H_
#define B200TBE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200TBE_API __attribute__((visibility("default")))
#else
#define B200TBE_API
#endif

/* A cudaStream_t, spelled without the CUDA headers. */
typedef struct CUstream_st* b200tbe_stream_t;

typedef enum {
  B200TBE_OK = 0,
  B200TBE_ERR_BAD_ARG = -1,       /* null pointer, negative size, unsupported combination */
  B200TBE_ERR_SCRATCH = -2,       /* scratch missing or smaller than *_scratch_bytes() */
  B200TBE_ERR_LAUNCH = -3,        /* cudaGetLastError() after a launch was not cudaSuccess */
  B200TBE_ERR_UNSUPPORTED = -4,   /* dtype or shape outside what the kernels cover */
  B200TBE_ERR_TOO_LARGE = -5      /* a size exceeds a fixed capacity of the entry point */
} b200tbe_status;

/* Element types of embedding rows and outputs (FBGEMM SparseType numbering). */
typedef enum {
  B200TBE_FP32 = 0,
  B200TBE_FP16 = 1,
  B200TBE_INT8 = 2,
  B200TBE_INT4 = 3,
  B200TBE_INT2 = 4,
  B200TBE_BF16 = 5
} b200tbe_dtype;

typedef enum { B200TBE_POOL_SUM = 0, B200TBE_POOL_MEAN = 1, B200TBE_POOL_NONE = 2 } b200tbe_pooling;

typedef enum { B200TBE_OPT_SGD = 0, B200TBE_OPT_ROWWISE_ADAGRAD = 1 } b200tbe_optimizer;

/* Bits a kernel may OR into the optional device status word (int32). */
#define B200TBE_DEV_INDEX_OUT_OF_RANGE 1
#define B200TBE_DEV_OFFSETS_NOT_MONOTONE 2
#define B200TBE_DEV_UNSUPPORTED_SHAPE 4 /* a table's row is not whole 16-byte vectors */
#define B200TBE_DEV_WAIT_TIMEOUT 8      /* reserved: a bounded wait inside a kernel gave up (no kernel of
                                           this version waits on anything but its own loads) */

#define B200TBE_MAX_DESTS 16
#define B200TBE_MAX_JAGGED_DIMS 4

B200TBE_API const char* b200tbe_status_string(int status);
B200TBE_API int b200tbe_abi_version(void);

/* ------------------------------------------------------------------------------------------------
 * TBE forward over fp32 / fp16 tables (the forward half of
 * torch.ops.fbgemm.split_embedding_codegen_lookup_{sgd,rowwise_adagrad}_function).
 *
 * Bags are table-major: bag (t, b) has id t*B + b and pools rows indices[offsets[id] ..
 * offsets[id+1]) of table t. Row r of table t starts at element weights_offsets[t] + r*D_t of
 * dev_weights, D_t = D_offsets[t+1] - D_offsets[t]. The pooled vector of bag (t, b) is written to
 *     outputs[b / rows_per_dest] + (b % rows_per_dest) * output_stride + output_col_offset
 *         + D_offsets[t]                                     (all in output elements)
 * With num_dests = 1 and rows_per_dest = B this is the usual [B, total_D] matrix. With
 * num_dests = G the kernel scatters the batch over G buffers, which may be peer-mapped memory of
 * other GPUs: the table-wise-sharded exchange then happens inside the lookup kernel.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* dev_weights;          /* flat buffer of all tables, weights_dtype elements */
  const int64_t* weights_offsets;   /* [T] element offset of each table's row 0 */
  const int32_t* D_offsets;         /* [T+1] output column of each table */
  const int64_t* rows_per_table;    /* [T] or NULL; when given, indices are range-checked */
  const void* indices;              /* [N] int64 or int32 row ids */
  const void* offsets;              /* [T*B+1] same integer type as indices */
  const float* per_sample_weights;  /* [N] or NULL */
  void* outputs[B200TBE_MAX_DESTS]; /* destination buffers, output_dtype elements */
  int64_t output_stride;            /* elements between consecutive rows of a destination */
  int64_t output_col_offset;        /* first column used inside a destination row */
  int64_t rows_per_dest;            /* batch rows per destination (B when num_dests == 1) */
  int32_t num_dests;
  int32_t T;
  int32_t B;
  int32_t max_D;                    /* max over tables of D_t; every D_t must be a multiple of 4 */
  int32_t weights_dtype;            /* B200TBE_FP32 or B200TBE_FP16 */
  int32_t output_dtype;             /* B200TBE_FP32 or B200TBE_FP16 */
  int32_t index_bytes;              /* 8 (int64) or 4 (int32) */
  int32_t pooling_mode;             /* B200TBE_POOL_SUM or B200TBE_POOL_MEAN */
  int32_t* status;                  /* device int32 or NULL; B200TBE_DEV_* bits are OR-ed in */
} b200tbe_forward_params;

B200TBE_API int b200tbe_forward(const b200tbe_forward_params* p, b200tbe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Quantised inference forward (torch.ops.fbgemm.int_nbit_split_embedding_codegen_lookup_function).
 *
 * dev_weights is a byte buffer. Row r of table t starts at byte weights_offsets[t] + r*stride_t,
 * stride_t = round_up(header + D_t*bits/8, row_alignment). INT8 / INT4 / INT2 rows begin with a
 * 4-byte header {fp16 scale, fp16 bias} followed by the packed payload (element 2i of an INT4 row
 * in the low nibble of byte i); FP16 / FP32 rows have no header. Value of an element:
 * q * scale + bias, accumulated in fp32. Output addressing as in b200tbe_forward_params.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const uint8_t* dev_weights;
  const int64_t* weights_offsets;   /* [T] byte offsets */
  const uint8_t* weights_tys;       /* [T] b200tbe_dtype of each table */
  const int32_t* D_offsets;         /* [T+1] */
  const int64_t* rows_per_table;    /* [T] or NULL */
  const void* indices;
  const void* offsets;
  const float* per_sample_weights;  /* [N] or NULL */
  void* outputs[B200TBE_MAX_DESTS];
  int64_t output_stride;
  int64_t output_col_offset;
  int64_t rows_per_dest;
  int32_t num_dests;
  int32_t T;
  int32_t B;
  int32_t max_D;
  int32_t row_alignment;            /* bytes; 16 on GPU tables, 1 for CPU-packed tables */
  int32_t output_dtype;             /* B200TBE_FP32 or B200TBE_FP16 */
  int32_t index_bytes;
  int32_t pooling_mode;
  int32_t* status;
  uint32_t table_type_mask;         /* optional: bit (1 << b200tbe_dtype) set for every type some table
                                       has (0: unknown). Lets the call skip the kernel for the types
                                       that are absent. A table of a type outside the mask is not
                                       pooled. */
} b200tbe_nbit_forward_params;

B200TBE_API int b200tbe_nbit_forward(const b200tbe_nbit_forward_params* p, b200tbe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * TBE backward with the optimizer applied in place (the backward half of
 * torch.ops.fbgemm.split_embedding_codegen_lookup_{sgd,rowwise_adagrad}_function).
 *
 * Steps, all on `stream`: (1) every lookup gets its row id as key and its bag id as payload; (2) a
 * least-significant-digit radix sort of every table's lookups by row id; (3) groups of lanes walk
 * the sorted lookups, summing the gradient slices of each run of equal rows (a run that spans
 * several walks is first reduced piecewise, then combined in a fixed order, so results do not
 * depend on scheduling); (4) the row is updated once ("exact" semantics):
 *   SGD:              w -= lr * g
 *   row-wise Adagrad: m += mean_d(g_d^2);  w -= lr / (sqrt(m) + eps) * g
 * g is the summed gradient (divided by the bag length first when pooling_mode is MEAN, multiplied
 * by the lookup's per-sample weight when given). fp16 weights are written back round-to-nearest.
 *
 * grad_output is [B, grad_stride] (elements of grad_dtype); the slice of bag (t, b) starts at
 * column grad_col_offset + D_offsets[t].
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  void* dev_weights;                /* updated in place */
  const int64_t* weights_offsets;   /* [T] element offsets */
  const int32_t* D_offsets;         /* [T+1] */
  const int64_t* hash_size_cumsum;  /* [T+1] exclusive prefix sum of rows per table */
  const void* indices;
  const void* offsets;
  const float* per_sample_weights;  /* [N] or NULL */
  const void* grad_output;
  int64_t grad_stride;
  int64_t grad_col_offset;
  float* momentum1;                 /* row-wise Adagrad state, one float per row; NULL for SGD */
  const int64_t* momentum1_offsets; /* [T] element offset of each table's state */
  int64_t num_indices;              /* N; must equal offsets[T*B] */
  int32_t T;
  int32_t B;
  int32_t max_D;
  int32_t total_hash_size_bits;     /* bits needed for hash_size_cumsum[T] - 1; at most 40 */
  int32_t weights_dtype;            /* B200TBE_FP32 or B200TBE_FP16 */
  int32_t grad_dtype;               /* B200TBE_FP32 or B200TBE_FP16 */
  int32_t index_bytes;
  int32_t pooling_mode;
  int32_t optimizer;                /* b200tbe_optimizer */
  float learning_rate;
  float eps;
  void* scratch;                    /* device memory, 256-byte aligned */
  size_t scratch_bytes;
  int32_t* status;
  void* grad_ready_event;           /* optional cudaEvent_t (NULL: none). The call makes `stream` wait
                                       for it after linearise, sort and segmentation, just before the
                                       first kernel that reads grad_output, so a gradient exchange
                                       running on another stream overlaps the part of the backward
                                       that needs only the indices. */
  int64_t max_table_rows;           /* optional: rows of the largest table (0: unknown). The sort then
                                       covers only the bits of a row id inside one table instead of
                                       total_hash_size_bits; a table with more rows than this is
                                       flagged B200TBE_DEV_UNSUPPORTED_SHAPE and its excess rows are
                                       treated as out of range. */
} b200tbe_backward_params;

/* Scratch needed by b200tbe_backward for num_indices lookups in T tables with keys of
 * total_hash_size_bits bits and rows of at most max_D elements. */
B200TBE_API size_t b200tbe_backward_scratch_bytes(int64_t num_indices, int32_t total_hash_size_bits,
                                                  int32_t max_D, int32_t T);
B200TBE_API int b200tbe_backward(const b200tbe_backward_params* p, b200tbe_stream_t stream);

/* The sort of step (2) on its own: keys_in/vals_in are sorted by the low `key_bits` bits into
 * keys_out/vals_out (stable; bits above key_bits are carried along but not compared). key_bytes is
 * 4 or 8; payloads are 4 bytes. All four arrays hold n elements (n < 2^31) and must not alias; the
 * inputs are overwritten (they are the ping-pong buffer). */
B200TBE_API size_t b200tbe_radix_sort_scratch_bytes(int64_t n);
B200TBE_API int b200tbe_radix_sort_pairs(void* keys_in, uint32_t* vals_in, void* keys_out,
                                         uint32_t* vals_out, int64_t n, int32_t key_bytes,
                                         int32_t key_bits, void* scratch, size_t scratch_bytes,
                                         b200tbe_stream_t stream);

/* Segmented form: the n pairs are num_segments independent segments, segment s being positions
 * [seg_offsets[s], seg_offsets[s+1]) (device array of num_segments + 1 int32 or int64 values,
 * non-decreasing, last = n); every segment is sorted on its own, stable, by the low key_bits bits of
 * its 4-byte keys, and no pair leaves its segment. This is step (2) of b200tbe_backward, where a
 * segment is one table's lookups and the key a row id: the passes cover the bits of a row id only,
 * not those that tell tables apart. The plan (segments -> tiles) is built on the device; the host
 * never reads seg_offsets. Arrays as b200tbe_radix_sort_pairs. */
B200TBE_API size_t b200tbe_radix_sort_segments_scratch_bytes(int64_t n, int32_t num_segments);
B200TBE_API int b200tbe_radix_sort_segments(uint32_t* keys_in, uint32_t* vals_in, uint32_t* keys_out,
                                            uint32_t* vals_out, int64_t n, const void* seg_offsets,
                                            int32_t offset_bytes, int32_t num_segments,
                                            int32_t key_bits, void* scratch, size_t scratch_bytes,
                                            b200tbe_stream_t stream);

/* The same sort for callers that cannot allocate device memory when they call it -- a plain C or
 * C++ host with no tensor allocator to borrow scratch from, a server that has already given all of
 * HBM to its tables, a loop that cannot take the device-wide synchronisation of cudaMalloc. The
 * scratch is a fixed array inside the library (about 2 MiB on every GPU that loads it, held
 * until the process exits), so n is limited to b200tbe_radix_sort_pairs_static_max() = 2^20 pairs;
 * larger n returns B200TBE_ERR_TOO_LARGE. The entry point calls no cudaMalloc, cudaFree or other
 * allocating routine. Its first call on a device looks up the array's device address (once per
 * device, with that device current); make that first call before any stream capture begins.
 * All calls on a device share the array: two calls whose kernels can overlap on the GPU (different
 * streams without an ordering between them) race on it and must be serialised by the caller.
 * Nothing in the array needs clearing between calls. This entry point has no counterpart in
 * intel/torchlib-xpu or in fbgemm_gpu. Other arguments as b200tbe_radix_sort_pairs. */
B200TBE_API int64_t b200tbe_radix_sort_pairs_static_max(void);
B200TBE_API int b200tbe_radix_sort_pairs_static(void* keys_in, uint32_t* vals_in, void* keys_out,
                                                uint32_t* vals_out, int64_t n, int32_t key_bytes,
                                                int32_t key_bits, b200tbe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Row-wise min-max quantisation to INT8 / INT4 / INT2 with an fp16 {scale, bias} pair per row, and
 * back (torch.ops.fbgemm.FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf and
 * torch.ops.fbgemm.FusedNBitRowwiseQuantizedSBHalfToFloatOrHalf; arithmetic of FBGEMM
 * include/fbgemm/QuantUtils.h:277-308). scale = (max - bias) / (2^bits - 1) and bias = min, both
 * rounded to fp16 first; q = rint((x - bias) / scale), clamped; a zero range stores scale 1.
 * header_first = 1 gives the table layout b200tbe_nbit_forward reads (header, payload, padding to
 * row_alignment); header_first = 0 with row_alignment = 1 gives FBGEMM's op layout (payload, header).
 * src / dst of the float side are [rows, D] contiguous, src_dtype / dst_dtype FP32 or FP16.
 * ---------------------------------------------------------------------------------------------- */
B200TBE_API int64_t b200tbe_quantized_row_bytes(int32_t D, int32_t ty, int32_t row_alignment);
B200TBE_API int b200tbe_quantize_rows(const void* src, int32_t src_dtype, int64_t rows, int32_t D,
                                      int32_t ty, int32_t row_alignment, int32_t header_first,
                                      uint8_t* dst, b200tbe_stream_t stream);
B200TBE_API int b200tbe_dequantize_rows(const uint8_t* src, int64_t rows, int32_t D, int32_t ty,
                                        int32_t row_alignment, int32_t header_first, void* dst,
                                        int32_t dst_dtype, b200tbe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * NV12 -> packed RGB24, BT.709: replaces the reference plugin's only device kernel,
 * convertNV12ToRGB(queue, y_plane, uv_plane, rgb_output, width, height, stride, fullrange)
 * (packages/torchcodec-xpu/src/torchcodec_xpu/ColorConversionKernel.h:12-20, .cpp:160-181), called
 * from XpuDeviceInterface.cpp:448-456 on the decoded VAAPI surface with fullrange = false. Same argument meaning; the
 * stream replaces the SYCL queue and, unlike the reference (a blocking queue.wait()), the call does
 * not synchronise. y_plane / uv_plane: device pointers to the luma plane and the interleaved U,V
 * plane, `stride` bytes per row in both; rgb: [height, width, 3] bytes. tiled = 1 reads the Intel
 * Tile-Y layout the reference's surfaces have (stride a multiple of 128, plane heights padded to 32
 * rows); tiled = 0 reads linear-pitch planes (what a CUDA decoder produces). fullrange selects the
 * reference's second normalisation, restated as written there (.cpp:84-88).
 * ---------------------------------------------------------------------------------------------- */
B200TBE_API int b200tbe_nv12_to_rgb(const uint8_t* y_plane, const uint8_t* uv_plane, uint8_t* rgb,
                                    int32_t width, int32_t height, int32_t stride, int32_t fullrange,
                                    int32_t tiled, b200tbe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Gradient exchange of the table-wise-sharded configuration (the step a sharded caller runs between
 * its dense part and b200tbe_backward; the pooled rows travel the other way inside b200tbe_forward,
 * which can scatter into peer-mapped destination buffers), as a push, which is what NVLink prefers
 * (stores stream, loads wait): src is this rank's gradient matrix, rows x (num_dsts * block_bytes)
 * with rows src_stride_bytes apart; column block d of row r is stored at row dst_row_offset + r of
 * destination d's matrix (rows dst_stride_bytes apart, block_bytes wide; peer-mapped or local). Byte
 * counts and pointers are multiples of 16. The caller orders the call after the destinations'
 * previous readers and orders the destinations' next readers after it (stream-ordered barriers). No
 * counterpart in the reference.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* src;
  void* dsts[B200TBE_MAX_DESTS];
  int64_t src_stride_bytes;
  int64_t dst_stride_bytes;
  int64_t dst_row_offset;
  int64_t rows;
  int64_t block_bytes;
  int32_t num_dsts;
} b200tbe_exchange_push_params;

B200TBE_API int b200tbe_exchange_push(const b200tbe_exchange_push_params* p,
                                      b200tbe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Segment permutation of jagged data (the data movement of torch.ops.fbgemm.permute_2D_sparse_data
 * and of the input distribution of a table-wise sharded lookup, where ids arrive grouped by source
 * rank and are regrouped by table): out segment j = in segment perm[j].
 * in_offsets[num_segments + 1] are the starts of the input segments, out_offsets[num_segments + 1]
 * the starts of the output segments (the caller computes them as the exclusive sum of the permuted
 * lengths; out_offsets[num_segments] = total_elems). Elements are moved as raw bytes: elem_bytes 2,
 * 4 or 8 (ids, per-sample weights). offset_bytes and perm_bytes are 4 or 8. No counterpart in the
 * reference.
 * ---------------------------------------------------------------------------------------------- */
B200TBE_API int b200tbe_permute_segments(const void* in, void* out, const void* in_offsets,
                                         const void* out_offsets, const void* perm,
                                         int64_t num_segments, int64_t total_elems, int32_t elem_bytes,
                                         int32_t offset_bytes, int32_t perm_bytes,
                                         b200tbe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Jagged tensors. values is [total_rows, inner_size]; dense is [outer_size, max_lengths[0], ...,
 * max_lengths[n-1], inner_size]; offsets[d] is the d-th level's offsets array (offsets[0] has
 * outer_size + 1 entries). Elements are moved as raw bytes, so any dtype of elem_bytes 1, 2, 4 or 8
 * works for the two copies; the add supports fp32, fp16 and bf16.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* offsets[B200TBE_MAX_JAGGED_DIMS]; /* device arrays, int64 or int32 */
  int64_t max_lengths[B200TBE_MAX_JAGGED_DIMS];
  int32_t num_jagged_dims;          /* 1 .. B200TBE_MAX_JAGGED_DIMS */
  int32_t offset_bytes;             /* 8 or 4 */
  int64_t outer_size;               /* B */
  int64_t inner_size;               /* D, elements per row */
  int64_t total_rows;               /* rows of values */
  int32_t elem_bytes;
  int32_t dtype;                    /* b200tbe_dtype; used by the add only */
} b200tbe_jagged_shape;

/* torch.ops.fbgemm.jagged_to_padded_dense: dense[b, l.., :] = values[row(b, l..), :] or the
 * padding value (the low elem_bytes bytes of pad_bits) where the position is past a length. */
B200TBE_API int b200tbe_jagged_to_padded_dense(const b200tbe_jagged_shape* s, const void* values,
                                               void* dense, uint64_t pad_bits,
                                               b200tbe_stream_t stream);

/* torch.ops.fbgemm.dense_to_jagged: values[row(b, l..), :] = dense[b, l.., :] for every position
 * inside the lengths. Rows of values that no position maps to (lengths above max_lengths) are
 * zero-filled. */
B200TBE_API int b200tbe_dense_to_jagged(const b200tbe_jagged_shape* s, const void* dense,
                                        void* values, b200tbe_stream_t stream);

/* torch.ops.fbgemm.jagged_dense_elementwise_add: out = to_padded_dense(x_values, pad 0) + y. */
B200TBE_API int b200tbe_jagged_dense_elementwise_add(const b200tbe_jagged_shape* s,
                                                     const void* x_values, const void* y,
                                                     void* out, b200tbe_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200TBE_H_ */
