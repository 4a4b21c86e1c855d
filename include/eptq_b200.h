/*
 * eptq_b200 -- C ABI of the B200 (sm_100a) quantized-linear inference path.
 *
 * Plain C, no torch types: every pointer is a raw CUDA device pointer owned by
 * the caller, every size an int, `stream` a cudaStream_t passed as void*.
 * Calls are asynchronous on `stream`, never synchronise, never allocate or free
 * device memory and keep no pointer after they return.  Every function returns
 * an EptqStatus; eptq_strerror() turns it into text.
 *
 * The entry points replace the reference's pybind module `_eptq_cuda`
 * (csrc/binding.cpp:4-16) and the C++ functions behind it
 * (csrc/eptq_kernels.h:15-41, csrc/eptq_kernels.cu:466-579).
 */
#ifndef EPTQ_B200_H
#define EPTQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EPTQ_ABI_VERSION 3

typedef enum EptqStatus {
    EPTQ_OK = 0,
    EPTQ_ERR_NULL = 1,        /* a required pointer is null                         */
    EPTQ_ERR_SHAPE = 2,       /* M, N, B, qb_size or table size out of range        */
    EPTQ_ERR_ALIGN = 3,       /* a pointer is not aligned for 128-bit access        */
    EPTQ_ERR_QUANTIZER = 4,   /* quantizer id is neither EPTQ_E8 nor EPTQ_E8D4      */
    EPTQ_ERR_WORKSPACE = 5,   /* workspace missing or smaller than required         */
    EPTQ_ERR_LAUNCH = 6,      /* the CUDA runtime rejected a launch or set-up call  */
    EPTQ_ERR_UNSUPPORTED = 7, /* valid arguments, but no kernel covers them         */
    EPTQ_ERR_TIMEOUT = 8      /* a bounded device-side wait ran out                 */
} EptqStatus;

enum { EPTQ_E8 = 0, EPTQ_E8D4 = 1 };

/*
 * One quantized linear layer, as the reference stores it in
 * `QuantizedLayerData` (config.py:98-159) plus the side tables
 * `EPTQLinear.from_quantized_data` derives at load time
 * (kernels/linear.py:122-139).
 *
 *   Q          int16 (M, N) row-major, M = out_features/8, N = in_features.
 *              Stored value = codebook index - 32768; 32767 marks a critical
 *              block whose 8 values live in O_vals.
 *   table32    fp32 codebook already divided by the radius: E8 (table_rows, 8),
 *              E8-D4 (512, 4) = (4 classes, 128 codes, 4 dims) flattened.
 *              Needed for bit-exact reconstruction (eptq_dequantize, eptq_gemm).
 *   table16    the same table rounded to fp16 (what the reference's kernels
 *              read, kernels/linear.py:93-95).  Needed by the GEMV.
 *   table8     E8-D4 only, optional, HOST memory: the 512 codes as int8 lattice
 *              coordinates, 4 per code (table = coordinate * table8_scale), made by
 *              eptq_prepare_d4_table8.  The library copies the 2 KB into the kernel's
 *              parameters at each launch, so the buffer only has to live until the
 *              call returns.  Enables the streaming integer-tensor-core GEMV
 *              (batch 1, N a multiple of 64 and at most 27648, no group scales);
 *              NULL selects the fp16-table kernels.
 *   table_packed  E8 only, optional: the table as table_packed_scale * (half-integer
 *              lattice coordinates), one 32-bit word per entry, 65536 words (entry
 *              65535 = the zero vector).  Coordinate c of dimension d is stored as
 *              n = 2c + 6 (0..12) in a 4-bit field at bit 2 + 4*f(d) with
 *              f = {0, 4, 1, 5, 2, 6, 3, 7} for d = 0..7; the last field wraps
 *              around (its low two bits are bits 31:30, its high two bits 1:0).
 *              Enables the persistent tensor-core GEMV for E8 layers; NULL selects
 *              the general kernel.  A table that is not such a multiple (a radially
 *              warped codebook) has no packed form.
 *   g, h       fp16 row scales (8*M) and column scales (N).
 *   O_vals     fp16 (n_masked, 8), ordered by row-major position of the markers.
 *   O_col      int32 (n_masked) column of each marker, same order.
 *   O_row_ptr  int32 (M+1) CSR row pointers into O_vals / O_col.
 *   crit_ptr, crit_pos, crit_O   optional side table of the same kind as O_col / O_row_ptr, derived at load
 *              time: the critical blocks grouped by the 64-row x 128-column unit of Q
 *              they fall into, units in row-tile-major order (unit = (row/64) *
 *              ceil(N/128) + col/128).  crit_ptr int32 (units + 1) offsets; crit_pos
 *              uint32 (n_masked) = (row % 64) << 16 | col; crit_O fp16 (n_masked, 8) =
 *              O_vals in that order.  With it the streaming GEMV patches critical blocks
 *              in step with the index stream instead of walking the CSR; all three NULL
 *              otherwise.  The kernel sums a row's corrections in 32-bit fixed point:
 *              pass the lists only if, for every Q row and each of the 8 dimensions, the
 *              sum over the row's critical blocks of (|O| + max|code|) / table8_scale stays
 *              below 3900 (the Python module checks this and falls back to the CSR tables).
 *   bias       fp16 (8*M) or NULL.
 *   S_group    fp16 (8*M/qb_size, N) group scales or NULL (then qb_size = 0).
 *              qb_size must be a multiple of 8.
 */
typedef struct EptqLayer {
    int32_t quantizer;        /* EPTQ_E8 or EPTQ_E8D4 */
    int32_t M;
    int32_t N;
    int32_t n_masked;         /* rows of O_vals; -1 = not stated (read from O_row_ptr[M]) */
    int32_t qb_size;
    int32_t table_rows;       /* E8: rows of the table (<= 65535); E8-D4: 512 */
    const int16_t* Q;
    const float* table32;
    const uint16_t* table16;
    const uint16_t* g;
    const uint16_t* h;
    const uint16_t* O_vals;
    const int32_t* O_col;
    const int32_t* O_row_ptr;
    const uint16_t* bias;
    const uint16_t* S_group;
    const uint8_t* table8;
    float table8_scale;
    float h_absmax;           /* max |h|, or 0 if not known (then the persistent GEMV is not used) */
    const uint32_t* table_packed; /* E8 only, optional: 65536 packed entries, see below */
    float table_packed_scale;
    int32_t reserved;
    const int32_t* crit_ptr;
    const uint32_t* crit_pos;
    const uint16_t* crit_O;
} EptqLayer;

/* ABI version of the loaded library (EPTQ_ABI_VERSION at build time). */
int eptq_abi_version(void);

/* Text for a status code; never NULL. */
const char* eptq_strerror(int status);

/* Number of kernels this library has launched in the calling process since it
 * was loaded (all entry points, all streams).  For launch accounting only. */
uint64_t eptq_launch_count(void);
/* The same per kernel family, to tell which kernel a call reached. */
enum { EPTQ_KERNEL_GEMV_STREAM = 0, EPTQ_KERNEL_GEMV_GROUP = 1, EPTQ_KERNEL_GEMV_MMA = 2, EPTQ_KERNEL_GEMV_SIMT = 3,
       EPTQ_KERNEL_GEMM = 4, EPTQ_KERNEL_OTHER = 5, EPTQ_KERNEL_COUNT = 6 };
uint64_t eptq_kernel_launch_count(int kernel);

/*
 * Host-side, no GPU involved: express an E8-D4 table (512 x 4 fp32, already
 * divided by the radius, as the reference builds it in quantizers/e8_d4.py:83-86)
 * as scale * (integer lattice coordinates, twice the half-integer D4 coordinates)
 * and write the 2048 coordinates as int8 to `out`, the scale to `*scale`.  Returns
 * EPTQ_ERR_UNSUPPORTED when the table is not such a multiple (for example a
 * radially warped codebook); such layers run on the fp16-table kernels.
 */
int eptq_prepare_d4_table8(const float* table, uint8_t* out, float* scale);

/*
 * Bytes of device scratch eptq_linear_forward / eptq_e8_forward /
 * eptq_e8d4_forward may need for a layer of this shape at batch B.  The caller
 * allocates it once (256-byte aligned), zero-fills it once, and may reuse it
 * for every call that is ordered on one stream, for layers of any shape (take
 * the maximum of the sizes): the first 1 MiB holds counters and accumulators
 * that every kernel returns to zero, the rest is overwritten before it is
 * read.  Calls that may overlap on the GPU need separate scratch.
 */
size_t eptq_workspace_bytes(int M, int N, int B);
/* The same from the layer itself: for prefill-sized B when the tensor-core GEMM takes the layer, the first
 * 1 MiB only (16 < B < 1024) or 1 MiB + 16*M*N bytes (B >= 1024: the fp16 weight is reconstructed once into the
 * scratch and a dense GEMM follows; with a smaller scratch the call still works and reconstructs tile by tile);
 * eptq_workspace_bytes(M, N, B) otherwise. */
size_t eptq_layer_workspace_bytes(const EptqLayer* layer, int B);

/*
 * Fused dequantise + matrix-vector product for decode, the replacement of
 * `e8_forward` (csrc/eptq_kernels.h:15-25, csrc/eptq_kernels.cu:563-570).
 * Same arguments with raw pointers: Q (M,N) int16; codebook fp16
 * (table_rows, 8); g (8M); h (N); x (B,N) fp16 contiguous; O_vals (n,8);
 * O_col (n); O_row_ptr (M+1); bias (8M) or NULL; y (B, 8M) fp16 written by the
 * call.  Unlike the reference there is no M % 4 restriction.
 */
int eptq_e8_forward(const int16_t* Q, const uint16_t* codebook, int table_rows,
                    const uint16_t* g, const uint16_t* h, const uint16_t* x,
                    const uint16_t* O_vals, const int32_t* O_col,
                    const int32_t* O_row_ptr, const uint16_t* bias,
                    uint16_t* y, int M, int N, int B,
                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * Same for the E8-D4 codebook, the replacement of `e8d4_forward`
 * (csrc/eptq_kernels.h:31-41, csrc/eptq_kernels.cu:572-579).  `codes` is the
 * fp16 (512, 4) table; an index unpacks as type = (idx>>14)&3, i = (idx>>7)&127,
 * j = idx&127 and decodes to [codes[type*128+i], codes[type*128+j]].
 */
int eptq_e8d4_forward(const int16_t* Q, const uint16_t* codes,
                      const uint16_t* g, const uint16_t* h, const uint16_t* x,
                      const uint16_t* O_vals, const int32_t* O_col,
                      const int32_t* O_row_ptr, const uint16_t* bias,
                      uint16_t* y, int M, int N, int B,
                      void* workspace, size_t workspace_bytes, void* stream);
/*
 * At batch 1 eptq_e8d4_forward runs the streaming kernel when `codes` is a multiple of the D4 lattice.  The
 * library finds that out the first time it sees a `codes` pointer outside a stream capture: it copies the
 * 4 KB table to the host (this first call synchronises) and remembers the answer for the pointer.  Make that
 * first call before capturing a graph; if the table behind a pointer is replaced, call
 * eptq_forget_codebook(pointer) (NULL forgets all).  eptq_linear_forward with table8_scale set needs none of
 * this and also takes the critical-block unit lists.  eptq_e8_forward has no such shortcut (its packed table
 * is 256 KB of device memory, which this library does not allocate): use eptq_linear_forward with
 * table_packed for E8 layers.
 */
void eptq_forget_codebook(const void* codes);

/*
 * Layer forward from the full descriptor: y (B, 8M) fp16 = x (B, N) fp16
 * through the quantized layer, including group scales (the reference has no
 * kernel for those and multiplies by a pre-reconstructed weight instead,
 * kernels/linear.py:97-120,159-164).  Chooses the decode GEMV or the
 * tensor-core GEMM from B alone.
 */
int eptq_linear_forward(const EptqLayer* layer, const uint16_t* x, uint16_t* y,
                        int B, void* workspace, size_t workspace_bytes,
                        void* stream);

/*
 * Forward of `n_layers` (1..32) independent layers in ONE launch: y[i] (B, 8*M_i)
 * = layer i applied to x[i] (B, N_i).  For layers whose inputs are all ready --
 * q/k/v or gate/up of a decoder layer (the reference calls them one by one,
 * kernels/linear.py:154-212), the experts of a mixture, or a single layer.
 * Requirements: layers of one codebook (E8-D4 sharing one table16, or E8 sharing
 * one table_packed), no group scales, N % 32 == 0, h_absmax set, B <= 16;
 * otherwise EPTQ_ERR_UNSUPPORTED (call eptq_linear_forward per layer instead).
 * One launch covers two batch rows; larger B is run as ceil(B/2) launches over
 * the same weights.  `xs` / `ys` are host arrays of device pointers.  Scratch as for eptq_linear_forward, size from
 * eptq_group_workspace_bytes.
 */
size_t eptq_group_workspace_bytes(const EptqLayer* layers, int n_layers, int B);
int eptq_linear_forward_group(const EptqLayer* layers, int n_layers,
                              const uint16_t* const* xs, uint16_t* const* ys, int B,
                              void* workspace, size_t workspace_bytes, void* stream);

/*
 * The same launch with work fused around each layer (decode-step glue; the
 * reference leaves it to the HuggingFace forward, bench_decode.py:44-71).
 * `fusions` has one entry per layer, or is NULL (then identical to
 * eptq_linear_forward_group).
 *
 *   x_op  EPTQ_X_PLAIN    x is used as given.
 *         EPTQ_X_RMSNORM  the layer sees x * rsqrt(mean(x^2) + norm_eps) per batch
 *                         row (the column weight of the norm is expected folded
 *                         into h by the caller).  All layers or none; they must
 *                         share one x pointer, N and norm_eps.
 *   y_op  EPTQ_Y_STORE         y (B, 8M) = out
 *         EPTQ_Y_ADD_RESIDUAL  y = residual + out, both rounded to fp16 as two
 *                              separate ops would; residual may be y itself.
 *         EPTQ_Y_ROPE          rotary embedding on heads of 128 outputs (pairs
 *                              (i, i+64), angle = *position * inv_freq[i], cos/sin
 *                              times rope_scaling rounded to fp16), stored to y.
 *         EPTQ_Y_ROPE_TO_CACHE the same, stored into a key cache: y points to fp16
 *                              (B, 8M/128, max_len, 128), row *position.
 *         EPTQ_Y_TO_CACHE      no rotation, stored into a value cache likewise.
 *   The three head-wise ops need 8M a multiple of 128 (M % 16 == 0).  Fusions need B <= 2.
 */
enum { EPTQ_X_PLAIN = 0, EPTQ_X_RMSNORM = 2, EPTQ_X_SILU_MUL = 3 };
enum { EPTQ_Y_STORE = 0, EPTQ_Y_ADD_RESIDUAL = 1, EPTQ_Y_ROPE = 2, EPTQ_Y_ROPE_TO_CACHE = 3, EPTQ_Y_TO_CACHE = 4 };

typedef struct EptqFusion {
    int32_t x_op;
    int32_t y_op;
    float norm_eps;
    float rope_scaling;
    int32_t max_len;
    int32_t reserved;
    const uint16_t* residual;   /* fp16 (B, 8M) */
    const int64_t* position;    /* device scalar */
    const float* inv_freq;      /* device, 64 entries */
    const uint16_t* x_aux;      /* EPTQ_X_SILU_MUL: second input, fp16 (B, N) */
} EptqFusion;

int eptq_linear_forward_group_fused(const EptqLayer* layers, int n_layers, const EptqFusion* fusions,
                                    const uint16_t* const* xs, uint16_t* const* ys, int B,
                                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * Chained launch (no counterpart in the reference, which launches one kernel per
 * layer): like eptq_linear_forward_group_fused, but the layers are ordered in
 * phases (phases[i] non-decreasing from 0, steps of at most 1) and a layer of
 * phase k+1 may take as x (or x_aux, or residual) what a layer of phase k wrote --
 * o_proj, then gate/up on the updated residual stream, then down on
 * silu(gate)*up, in ONE launch.  Inside the launch every phase is spread over
 * all SMs and the weight stream of the next phase is prefetched while the last
 * tiles of the previous one are finished.
 *   x_op EPTQ_X_SILU_MUL: the layer sees silu(x) * x_aux, both (B, N) fp16,
 *   with the fp16 roundings of two separate operations (only in chained launches).
 *   EPTQ_X_RMSNORM may differ from layer to layer here.
 * Requirements: the streaming kernel's (E8-D4 with table8, batch 1, N % 64 == 0,
 * no group scales).  The launch is cooperative: it needs all SMs of the device
 * and fails with EPTQ_ERR_LAUNCH if they cannot all hold a block.  Every wait
 * inside is bounded (2 s); eptq_workspace_status tells whether one ran out.
 */
int eptq_linear_forward_chain(const EptqLayer* layers, int n_layers, const EptqFusion* fusions,
                              const int* phases, const uint16_t* const* xs, uint16_t* const* ys,
                              int B, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The last counter word of a scratch buffer is its status word: a kernel whose
 * bounded device-side wait ran out (the chained and streaming GEMV, the prefill
 * GEMM) leaves EPTQ_ERR_TIMEOUT there and its output is not valid.  This copies
 * the word to *host_out on `stream`, waits for that copy (it synchronises the
 * stream: do not call it during capture) and clears the word.
 */
int eptq_workspace_status(void* workspace, int* host_out, void* stream);

/*
 * Reconstruct the fp16 weight (8M, N) row-major, bit-for-bit what the
 * reference's `dequantize_layer` returns (algorithms/eptq.py:406-471):
 * table32 value (or the critical block from O_vals, which skips the group
 * scale), times S_group, times g, times h, each an fp32 multiply in that
 * order, one round-to-nearest-even to fp16.
 */
int eptq_dequantize(const EptqLayer* layer, uint16_t* W, void* stream);

/*
 * (No counterpart in the reference.)  Decode GEMV for callers that cannot
 * allocate device memory and therefore cannot provide the scratch buffer of
 * eptq_linear_forward -- a server whose memory is fully pre-reserved, a plug-in
 * that must stay out of its host's allocator, a loop that may not call an
 * allocator at all.  Same result as eptq_linear_forward; the scratch is a fixed
 * array of eptq_static_scratch_bytes() (4 MiB) inside the library's device
 * image, held by every GPU that loads the library until the process exits.
 *
 * Limits: E8-D4 layers without group scales, in_features a multiple of 32,
 * batch 1..4, and a scratch need of at most eptq_static_scratch_bytes()
 * (eptq_workspace_bytes tells the need); anything else returns
 * EPTQ_ERR_UNSUPPORTED or, for the size, EPTQ_ERR_WORKSPACE.  The call itself
 * never allocates or frees.  All calls on a device share the one array, which
 * keeps the previous call's contents: calls that may overlap on the GPU race,
 * so keep them ordered on one stream.  The first call on each device looks up
 * the array's address; make that first call before any stream capture.
 */
size_t eptq_static_scratch_bytes(void);
int eptq_linear_forward_static_scratch(const EptqLayer* layer, const uint16_t* x,
                                       uint16_t* y, int B, void* stream);

/*
 * Decode-step glue (the elementwise work between the quantized linears of a
 * LLaMA-style decoder layer).  The reference leaves these to the HuggingFace
 * forward and to torch.compile (bench_decode.py:44-71,149); they are part of
 * this ABI so that one decoded token is a short, fixed list of launches.
 * All tensors fp16, contiguous, 16-byte aligned.
 *
 * eptq_add_rmsnorm: for each of `rows` rows of length H (multiple of 8):
 *   if delta != NULL, x += delta (in place, rounded to fp16); then
 *   out = weight * fp16(x * rsqrt(mean(x^2) + eps))  (LlamaRMSNorm's roundings).
 * eptq_silu_mul: out[i] = fp16(fp16(silu(gate[i])) * up[i]), n a multiple of 8.
 * eptq_rope_append: token row r = b*T + t has cache position positions[t]
 *   (int64, device).  Rotates q (B*T, n_heads*head_dim) in place, writes the
 *   rotated k (B*T, n_kv_heads*head_dim) and v into the caches
 *   (B, n_kv_heads, max_len, head_dim) at that position.  Pairs (i, i+head_dim/2),
 *   angle = position * inv_freq[i] (fp32, device, head_dim/2 entries), cos/sin
 *   times `scaling` rounded to fp16.  Positions outside [0, max_len) are skipped.
 * eptq_decode_attention: out (B*T, n_heads*head_dim) = softmax(scale * q K^T) V
 *   over the cache positions 0..positions[t] of the row's batch entry; grouped
 *   key/value heads when n_kv_heads < n_heads.  head_dim 64 or 128, else
 *   EPTQ_ERR_UNSUPPORTED.  Meant for a few query tokens (decode); scratch of
 *   eptq_attention_workspace_bytes(B*T, n_heads, head_dim, max_len) bytes,
 *   256-byte aligned, zero-filled once, reusable by calls of any shape that are
 *   ordered on one stream (take the largest size).  Long contexts are split over
 *   several blocks per (row, head); that needs B*T*n_heads <= 16384.
 */
int eptq_add_rmsnorm(uint16_t* x, const uint16_t* delta, const uint16_t* weight,
                     uint16_t* out, int rows, int H, float eps, void* stream);
int eptq_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out,
                  size_t n, void* stream);
int eptq_rope_append(uint16_t* q, const uint16_t* k, const uint16_t* v,
                     uint16_t* k_cache, uint16_t* v_cache, const int64_t* positions,
                     const float* inv_freq, int B, int T, int n_heads, int n_kv_heads,
                     int head_dim, int max_len, float scaling, void* stream);
size_t eptq_attention_workspace_bytes(int rows, int n_heads, int head_dim, int max_len);
int eptq_decode_attention(const uint16_t* q, const uint16_t* k_cache,
                          const uint16_t* v_cache, const int64_t* positions,
                          uint16_t* out, int B, int T, int n_heads, int n_kv_heads,
                          int head_dim, int max_len, float scale, void* workspace,
                          size_t workspace_bytes, void* stream);

/*
 * Un-quantized output projection fused with the greedy pick.  The reference keeps
 * lm_head in fp16 (quantize.py:86-90) and picks the token from the logits of a
 * library GEMM (bench_decode.py:35-41).  W fp16 (V, H) row-major, x fp16 (B, H);
 * tokens[b] = first index of the maximum of fp16(W x_b), int64 on the device.
 * `norm_weight` (fp16 (H), or NULL) applies the model's final RMSNorm to x on the way
 * in: x_b <- norm_weight * fp16(x_b * rsqrt(mean(x_b^2) + eps)).  `logits` (fp16
 * (B, V), or NULL) also receives the logits.  H a multiple of 256 up to 8192, B <= 4.
 * Scratch: eptq_lm_head_workspace_bytes(B) bytes, 256-byte aligned, zero-filled once.
 */
size_t eptq_lm_head_workspace_bytes(int B);
int eptq_lm_head_argmax(const uint16_t* W, const uint16_t* x, const uint16_t* norm_weight, float eps,
                        uint16_t* logits, int64_t* tokens, int V, int H, int B, void* workspace,
                        size_t workspace_bytes, void* stream);

/*
 * (No counterpart in the reference, which is single-GPU.)  One-shot all-reduce (sum)
 * of a small fp16 vector over the GPUs of one node, for the partial outputs of
 * row-parallel layers in tensor-parallel decode.  Each rank owns a data buffer of
 * eptq_allreduce_data_bytes(n_ranks, n_max) bytes and a flag buffer of
 * eptq_allreduce_flag_bytes(n_ranks) bytes, both zero-filled once and mapped into
 * every peer (CUDA IPC or any other peer mapping; the caller's job).  `peer_data` /
 * `peer_flags` are host arrays of n_ranks device pointers, entry r = rank r's buffer
 * as seen from this GPU (entry `rank` = the local one).  Every rank calls with the
 * same n (multiple of 8, <= n_max) in the same order; `out` may be `x`.  With
 * `residual` (or NULL) the result is residual + sum, and `out` may be `residual`: the
 * residual stream of a decoder layer is updated by the reduction itself.  The kernel
 * stores its vector into every peer's buffer (plain 8-byte stores over NVLink, each
 * carrying two values and the call number), then polls -- bounded -- its own buffer
 * until every peer's words are there and sums locally.  A wait that runs out sets the
 * int that follows the call counters at the end of the local flag buffer to
 * EPTQ_ERR_TIMEOUT and leaves `out` unwritten.  At most 8 ranks.
 */
size_t eptq_allreduce_data_bytes(int n_ranks, int n_max);
size_t eptq_allreduce_flag_bytes(int n_ranks);
int eptq_allreduce_push(const uint16_t* x, uint16_t* out, const uint16_t* residual, int n,
                        void* const* peer_data, void* const* peer_flags, int rank, int n_ranks,
                        int n_max, void* stream);
/* Limit of that wait for later calls, in nanoseconds (0 = the default, two seconds).  Process-wide; meant
 * for tests that make the wait run out. */
void eptq_allreduce_set_wait_ns(unsigned long long ns);

#ifdef __cplusplus
}
#endif
#endif /* EPTQ_B200_H */
