/* scn_b200 -- C ABI of the B200 (sm_100a) forward path for spatially-sparse CNNs.
 *
 * Every entry point is the device-side replacement of one piece of the forward
 * (inference) path of btgraham/SparseConvNet-archived; the comment above each declaration
 * names the reference interface it replaces (paths inside the reference project,
 * SparseConvNet/...).  The C++ classes that keep the reference's names
 * (sparseconvnet-archived_b200/csrc/host/) call nothing but these functions.
 *
 * Conventions
 *   - all pointers named d_* are DEVICE pointers owned by the caller; nothing here
 *     allocates or frees device memory unless its comment says so;
 *   - `stream` is a cudaStream_t passed as an opaque pointer; calls enqueue work and
 *     return without synchronising unless stated;
 *   - every function returns an scn_status; nothing prints or exits (the reference
 *     prints and calls exit(), utilities.h:32-67);
 *   - rows ("spatial sites") are numbered across the whole batch; sample b owns the
 *     contiguous rows [off[b], off[b+1]) (BatchProducer.cu:54-58);
 *   - a grid is carried as `keys[row]`: the row-major site index inside the sample's
 *     S^dim cube (Regions.cu:195-200), or -1 for the sample's background ("null vector")
 *     row; `bg[b]` is that row's id (SparseGrid::backgroundCol, SparseGrid.h:68-77) or -1.
 */
#ifndef SCN_B200_H
#define SCN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *scn_stream_t; /* cudaStream_t */

enum scn_status {
  SCN_OK = 0,
  SCN_ERR_INVALID = 1,     /* bad argument (sizes, null pointers, unsupported geometry)   */
  SCN_ERR_CUDA = 2,        /* a CUDA runtime call or launch failed; see scn_last_error()   */
  SCN_ERR_WORKSPACE = 3,   /* workspace too small                                          */
  SCN_ERR_UNSUPPORTED = 4  /* valid in the reference, not built here                       */
};

/* Bits a rule-build kernel may set in d_result[2] (read them after the stream has run). */
#define SCN_DEV_ERR_CAPACITY 1  /* more output rows than rows_out_capacity: outputs truncated */
#define SCN_DEV_ERR_KEY 2       /* a key outside [0, nIn^dim) was skipped                      */
#define SCN_DEV_ERR_DUPLICATE 4 /* the same key twice in one sample                            */

/* ActivationFunction, types.h:20-29 (same numeric values). */
enum scn_activation {
  SCN_NOSIGMOID = 0, SCN_RELU = 1, SCN_VLEAKYRELU = 2, SCN_LEAKYRELU = 3,
  SCN_TANH = 4, SCN_SOFTMAX = 5, SCN_PRELU = 6, SCN_SIGMOID = 7
};

/* Arithmetic of the fused conv/NiN kernel. */
enum scn_precision {
  SCN_PREC_AUTO = -1,  /* tensor cores when the shape allows, else SIMT                    */
  SCN_PREC_FP32 = 0,   /* fp32 FMA on CUDA cores                                           */
  SCN_PREC_3XTF32 = 1, /* tcgen05 kind::tf32, hi/lo split of both operands (fp32-grade)    */
  SCN_PREC_BF16 = 2,   /* tcgen05 kind::f16 with bf16 operands, fp32 accumulation          */
  SCN_PREC_3XBF16 = 3, /* kind::f16, bf16 hi/lo split of both operands, three products     */
  SCN_PREC_SPLIT = 4   /* the three-product hi/lo split with the operand format chosen per
                          layer: bf16 (16 mantissa bits per product, half the tensor time)
                          where the kernel feeds A from tensor memory (fs*nIn >= 128), tf32
                          (21 bits) elsewhere; what SCN_PREC_AUTO resolves to by default    */
};
/* The tensor-core precision SCN_PREC_AUTO resolves to when the shape has a tensor-core path
 * (the host classes pack their weights for it).  No reference counterpart. */
int scn_conv_auto_precision(void);

#define SCN_LATTICE_SQUARE 0     /* RegularSquareRegions, Regions.cu:13-29      */
#define SCN_LATTICE_TRIANGULAR 1 /* RegularTriangularRegions, Regions.cu:804-832 */

/* The arguments of the reference's region constructors plus gridRules' minActiveInputs:
 * 1 = every touched output site, >1 = keep sites with at least that many active inputs,
 * -1 = 'valid' 3^dim convolution (square lattice). */
typedef struct {
  int lattice, dim, nIn, nOut, size, stride, minActive;
} scn_regions_t;

const char *scn_status_string(int status);
/* Message of the last failing call on this thread ("" if none). */
const char *scn_last_error(void);
/* Kernels this library has launched in this process so far (memsets and copies are not
 * counted).  No reference counterpart: the benchmark reports it. */
long long scn_kernel_launch_count(void);
/* 1 when the library was built for, and the current device is, compute capability 10.x. */
int scn_device_supported(void);

/* Cells per rule row: size^dim, or triangleSize(size, dim) (utilities.cu:14-32). */
int scn_regions_cells(const scn_regions_t *r);

/* Replaces gridRules() looped over a batch, i.e. the body of
 * ConvolutionalLayer::preprocess (ConvolutionalLayer.cu:101-123),
 * MaxPoolingLayer::preprocess (MaxPoolingLayer.cu:104-119),
 * ConvolutionalTriangularLayer::preprocess (ConvolutionalTriangularLayer.cu:23-45) and
 * MaxPoolingTriangularLayer::preprocess, with the builders of Regions.cu:338-526
 * (square Min), 528-653 (square NoMin), 658-780 (Valid), 834-970 and 972-1164
 * (triangular), and the SparseGrid/vectorHash maps they use (SparseGrid.h, vectorHash.cpp).
 * Output rows are numbered exactly as the reference's ascending-key (vectorHash) backend
 * numbers them; rule cells without an active input hold d_in_bg[b].
 *
 *   d_in_keys[rows_in], d_in_off[batch+1], d_in_bg[batch]   the input grids
 *   rows_in_bound   >= d_in_off[batch]; sizes the launches and the workspace
 *   d_out_keys[rows_out_capacity], d_out_off[batch+1], d_out_bg[batch]  the output grids
 *   d_rules[rows_out_capacity * scn_regions_cells(r)]
 *   d_result[4]     {output rows incl. background rows, output sites, SCN_DEV_ERR_* bits,
 *                    largest number of sites in one output sample}
 * No host synchronisation: the caller reads d_result when it needs the counts. */
size_t scn_rules_workspace_bytes(const scn_regions_t *r, int batch, int rows_in_bound);
int scn_rules_build(const scn_regions_t *r, int batch, const int *d_in_keys, const int *d_in_off,
                    const int *d_in_bg, int rows_in_bound, int *d_out_keys, int *d_out_off,
                    int *d_out_bg, int *d_rules, int rows_out_capacity, int *d_result,
                    void *d_workspace, size_t workspace_bytes, scn_stream_t stream);

/* Rules of a fractional max-pooling layer: FractionalPoolingRegions<ticks> (Regions.cu:127-157)
 * with gridRulesOverlappingNoMin (528-653) for the overlapping kinds and gridRulesNonOverlapping
 * (159-336) for the others, as the four FMP layers' preprocess() call them
 * (MaxPoolingLayer.cu:171-186, 232-247, 293-308, 354-369).  The tick tables are drawn on the host
 * (one FractionalPoolingRegions per sample, one ticks object per axis) and passed as
 * d_ticks[(b*dim + axis) * (2*nOut + 2*nIn)] = inputL[nOut], inputR[nOut], outputL[nIn], outputR[nIn].
 * Rule rows have poolSize^dim cells; in the non-overlapping case cells beyond a region hold -1.
 * All other arguments as scn_rules_build. */
size_t scn_fmp_rules_workspace_bytes(int dim, int nIn, int nOut, int poolSize, int batch, int rows_in_bound);
int scn_fmp_rules_build(int dim, int nIn, int nOut, int poolSize, int overlapping, int batch, const int *d_ticks,
                        const int *d_in_keys, const int *d_in_off, const int *d_in_bg, int rows_in_bound,
                        int *d_out_keys, int *d_out_off, int *d_out_bg, int *d_rules, int rows_out_capacity,
                        int *d_result, void *d_workspace, size_t workspace_bytes, scn_stream_t stream);

/* Replaces the loop "for every layer: layer->preprocess(batch, in, out)" of
 * BatchProducer::preprocessBatch (BatchProducer.cu:72-75) for the geometry layers
 * (convolutions and poolings, in network order) with ONE kernel: each sample's whole chain
 * of grids is built by one CTA in shared memory.  Only for small samples
 * (scn_rules_chain_supported says whether these layers and this per-sample row bound fit);
 * larger ones are built layer by layer with scn_rules_build.  Outputs per layer are exactly
 * those of scn_rules_build; layer l+1 reads layer l's output grid.
 *   max_rows_per_sample   upper bound on the rows (sites + background row) of one input sample
 *   rows_hint             0, or the largest number of rows one sample is expected to have in
 *                         any layer (e.g. 1.25 x what d_result[3] reported for earlier
 *                         batches): shared memory is sized for it instead of the worst case,
 *                         more samples run per SM, and a sample that exceeds it sets
 *                         SCN_DEV_ERR_CAPACITY (rebuild with rows_hint = 0). */
typedef struct {
  scn_regions_t regions;
  int *d_out_keys, *d_out_off, *d_out_bg, *d_rules; /* as in scn_rules_build */
  int rows_out_capacity;
  int *d_result; /* [4] as in scn_rules_build */
} scn_chain_layer_t;
size_t scn_rules_chain_workspace_bytes(int n_layers, int batch);
int scn_rules_chain_supported(const scn_chain_layer_t *layers, int n_layers, int batch, int max_rows_per_sample,
                              int rows_hint);
int scn_rules_chain_build(const scn_chain_layer_t *layers, int n_layers, int batch, const int *d_in_keys,
                          const int *d_in_off, const int *d_in_bg, int max_rows_per_sample, int rows_hint,
                          void *d_workspace, size_t workspace_bytes, scn_stream_t stream);

/* The same build for a caller that keeps the workspace to itself from one call to the next (a
 * network that processes batch after batch).  In steady state the kernel is the only stream
 * operation: layer descriptors stay on the device while they do not change, and every launch
 * prepares the per-sample counters, the ticket and the result records of the launch AFTER
 * it, which stream order puts behind it.  No reference counterpart.
 *   st              host-side bookkeeping from scn_rules_chain_resident_create (no device memory);
 *                   scn_rules_chain_resident_invalidate after anything else wrote the workspace
 *   d_workspace     scn_rules_chain_resident_workspace_bytes(n_layers, batch) bytes that nothing
 *                   else writes between calls
 *   phase           0 or 1, alternating from call to call; the layers' d_result records belong
 *                   to this phase
 *   d_result_next   a block of n_result_next ints that holds every d_result record the NEXT
 *                   call (other phase) will name, cleared by this launch; NULL if the next
 *                   call is not known to be a resident one
 *   d_in_bg         may be NULL: every sample's background row (the row with a negative key,
 *                   -1 if none) is then found by the kernel and written to d_in_bg_out[batch]. */
typedef struct scn_chain_resident scn_chain_resident_t;
scn_chain_resident_t *scn_rules_chain_resident_create(void);
void scn_rules_chain_resident_destroy(scn_chain_resident_t *st);
void scn_rules_chain_resident_invalidate(scn_chain_resident_t *st);
size_t scn_rules_chain_resident_workspace_bytes(int n_layers, int batch);
int scn_rules_chain_build_resident(scn_chain_resident_t *st, const scn_chain_layer_t *layers, int n_layers, int batch,
                                   const int *d_in_keys, const int *d_in_off, const int *d_in_bg, int *d_in_bg_out,
                                   int max_rows_per_sample, int rows_hint, void *d_workspace, size_t workspace_bytes,
                                   int phase, int *d_result_next, int n_result_next, scn_stream_t stream);

/* scn_rules_build for callers that cannot allocate device memory (no counterpart in the
 * reference, whose rule construction runs on the host).  Hosts embedded in a framework that
 * owns the GPU's memory, code on a latency-critical path that must stay clear of cudaMalloc
 * (it can lock and synchronise the whole device), or a plugin loaded after a pool has taken
 * all free memory still pass their own input and output buffers, but the scratch comes from a
 * fixed array of SCN_RULES_STATIC_SCRATCH_BYTES compiled into the library; each GPU that loads
 * the library keeps that much memory reserved until the process exits.  The call allocates and
 * frees nothing.  Arguments and results are those of scn_rules_build without the workspace.
 *   - A build whose scn_rules_workspace_bytes() exceeds the array is refused with
 *     SCN_ERR_WORKSPACE and a message naming both sizes.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress): make that first call outside any stream capture.
 *   - All calls on a device share the one array.  It keeps the last call's contents and the
 *     kernels clear what they need cleared, so back-to-back calls on one stream are fine;
 *     calls that can overlap on the GPU (different streams, different threads) race and
 *     corrupt each other's rules.
 *   - The array's device address is looked up once per device ordinal and kept for the life of
 *     the process: it does not survive cudaDeviceReset() or a second context on that ordinal. */
#define SCN_RULES_STATIC_SCRATCH_BYTES (16u << 20)
size_t scn_rules_static_scratch_bytes(void);
int scn_rules_build_static(const scn_regions_t *r, int batch, const int *d_in_keys, const int *d_in_off,
                           const int *d_in_bg, int rows_in_bound, int *d_out_keys, int *d_out_off,
                           int *d_out_bg, int *d_rules, int rows_out_capacity, int *d_result,
                           scn_stream_t stream);

/* Replaces terminalGridPoolingRules() looped over a batch (TerminalPoolingLayer.cu:8-20,
 * 81-99): row b lists sample b's rows in ascending key order (its background row if it has
 * no site), padded with -1 to S columns; the output grid is one site (key 0) per sample.
 * S must be >= the largest site count of a sample (the reference uses max(1, that)).
 * `spatial_size`^dim bounds the keys.  d_result as above. */
size_t scn_terminal_rules_workspace_bytes(int dim, int spatial_size, int batch, int rows_in_bound);
int scn_terminal_rules_build(int dim, int spatial_size, int batch, const int *d_in_keys,
                             const int *d_in_off, const int *d_in_bg, int rows_in_bound, int S,
                             int *d_out_keys, int *d_out_off, int *d_out_bg, int *d_rules,
                             int *d_result, void *d_workspace, size_t workspace_bytes,
                             scn_stream_t stream);

/* Replaces ConvolutionalLayer::forwards + NetworkInNetworkLayer::forwards (test branch) as
 * ONE kernel: propForwardToMatrixMultiply (ConvolutionalLayer.cu:12-41, 124-133), then
 * replicateArray + cublasSgemm(alpha=p, beta=p) + applySigmoid
 * (NetworkInNetworkLayer.cu:187-201; SigmoidLayer.cu:187-222), or dPReLU
 * (NetworkInNetworkPReLULayer.cu:8-23, 159-170):
 *     out[r][n] = act( p * sum_{f,c} in[rules[r*fs+f]][c] * W[(f*nIn+c)*N + n] + p * B[n] )
 * d_rules == NULL (then fs must be 1) is a plain NetworkInNetworkLayer.  A negative rule
 * contributes a zero row.  d_prelu (per-channel slopes) is required iff act == SCN_PRELU.
 * act == SCN_SOFTMAX applies the row softmax of SigmoidLayer.cu:160-177 (N <= 1024).
 * `precision` is an scn_precision; shapes a tensor-core path cannot take return
 * SCN_ERR_UNSUPPORTED unless SCN_PREC_AUTO.  d_W_packed is the result of
 * scn_conv_pack_weights for that precision, or NULL for SCN_PREC_FP32. */
int scn_conv_nin_forward(const float *d_in, const int *d_rules, int rows_out, int fs, int nIn,
                         const float *d_W, const void *d_W_packed, const float *d_B,
                         const float *d_prelu, int N, float p, int act, int precision,
                         float *d_out, scn_stream_t stream);
/* The same with optional scratch: layers with few output tiles (small rows_out, large K) then
 * split K over several CTAs per tile, write partial sums to the scratch and finish with a
 * second small kernel (summed in a fixed order: results stay deterministic).
 * scn_conv_nin_workspace_bytes() is the size worth passing (0: the layer does not benefit). */
size_t scn_conv_nin_workspace_bytes(int rows_out, int fs, int nIn, int N, int precision);
int scn_conv_nin_forward_ws(const float *d_in, const int *d_rules, int rows_out, int fs, int nIn,
                            const float *d_W, const void *d_W_packed, const float *d_B,
                            const float *d_prelu, int N, float p, int act, int precision,
                            float *d_out, void *d_workspace, size_t workspace_bytes, scn_stream_t stream);

/* The same fused layer launched before the host knows the row count: rows_out_bound is an upper
 * bound (d_out and d_rules are sized for it), the kernel reads the count itself from *d_rows_out,
 * where an earlier call on the same stream (scn_rules_build's d_result[0], say) leaves it.  Split
 * tensor-core kernel only (precision SCN_PREC_3XTF32 or SCN_PREC_SPLIT, weights packed for it;
 * SCN_ERR_UNSUPPORTED for other shapes), no softmax.  It lets the first layer of a network start while the rulebooks' counts travel to the host.
 * No reference counterpart. */
int scn_conv_nin_forward_dyn(const float *d_in, const int *d_rules, int rows_out_bound, const int *d_rows_out,
                             int fs, int nIn, const void *d_W_packed, const float *d_B, const float *d_prelu,
                             int N, float p, int activation, float *d_out, int precision, scn_stream_t stream);

/* ConvolutionalLayer gather + NetworkInNetworkLayer + MaxPoolingLayer in one kernel (ConvolutionalLayer.cu:124-133,
 * NetworkInNetworkLayer.cu:187-201, MaxPoolingLayer.cu:9-35) for pooling windows that do not overlap
 * (poolStride == poolSize) and hold 2, 4, 8, 16 or 32 cells: the tile rows of the contraction are ordered
 * window by window (row d_pool_rules[w*cells + c] of the learnt layer's output), the epilogue takes the
 * maximum over each window (negative rules skipped, first maximum wins) and writes only
 * d_out[rows_pool x N] and d_choices (flat index rule*N + column); the learnt layer's own output never
 * reaches memory.  d_rules are the convolution's rules (fs cells per row).  d_rows_pool: NULL, or the
 * device-side row count (then rows_pool_bound is an upper bound).  rows_unpooled: rows of the learnt
 * layer's own output if known, else 0; with it the call also answers SCN_ERR_UNSUPPORTED where fusing would
 * cost an extra wave of tiles (windows repeat background rows) or where the layer alone would split K
 * and no workspace is given.  d_workspace (may be NULL): scn_conv_nin_workspace_bytes(rows_unpooled, ...)
 * bytes; with it (and rows_unpooled, and no d_rows_pool) a layer that splits K keeps doing so and the pooling
 * happens in the kernel that adds the partial sums.
 * Split tensor-core kernel only (precision SCN_PREC_3XTF32 or SCN_PREC_SPLIT, weights packed for it);
 * SCN_ERR_UNSUPPORTED for shapes it does not take. */
int scn_conv_nin_maxpool_forward(const float *d_in, const int *d_rules, int fs, int nIn, const void *d_W_packed,
                                 const float *d_B, const float *d_prelu, int N, float p, int activation,
                                 const int *d_pool_rules, int pool_cells, int rows_pool_bound, const int *d_rows_pool,
                                 int rows_unpooled, float *d_out, int *d_choices, void *d_workspace, size_t workspace_bytes,
                                 int precision, scn_stream_t stream);

/* Two learnt layers in a row where the first has few rows and a long K (the top of a network: ConvolutionalLayer
 * gather + NetworkInNetworkLayer, NetworkInNetworkLayer.cu:187-201, then the classifier's NetworkInNetworkLayer with
 * its softmax, SigmoidLayer.cu:160-177): the first runs on the 3xTF32 kernel with K split over several CTAs
 * (d_workspace: scn_conv_nin_workspace_bytes(rows_out, ...) bytes, must be > 0) and the kernel that adds the partial
 * sums also applies the second layer W2[N x N2] (fp32, N2 <= 16, softmax allowed).  d_mid[rows_out x N] receives the
 * first layer's output as scn_conv_nin_forward_ws would write it, d_out[rows_out x N2] the second's.
 * precision: SCN_PREC_3XTF32 or SCN_PREC_SPLIT (the first layer's packed weights are for it).
 * SCN_ERR_UNSUPPORTED where the first layer would not split K or the shapes do not fit: run the two layers. */
int scn_conv_nin_nin_forward(const float *d_in, const int *d_rules, int rows_out, int fs, int nIn, const void *d_W_packed,
                             const float *d_B, const float *d_prelu, int N, float p, int activation, const float *d_W2,
                             const float *d_B2, const float *d_prelu2, int N2, float p2, int activation2, float *d_mid,
                             float *d_out, void *d_workspace, size_t workspace_bytes, int precision, scn_stream_t stream);

/* One-time repack of W[K x N] (K = fs*nIn) for a tensor-core precision: bytes needed, then
 * the packing kernel.  No reference counterpart (the reference hands W to cuBLAS as is). */
size_t scn_conv_packed_weight_bytes(int K, int N, int precision);
int scn_conv_pack_weights(const float *d_W, int K, int N, int precision, void *d_W_packed,
                          scn_stream_t stream);

/* Every wait inside the tensor-core kernel has a time limit (2 s); a wait that runs out
 * records a code and the kernel proceeds to its normal exit.  Returns that code (0 = none)
 * and clears it; copies from the device, so it waits for running work.  No reference
 * counterpart. */
int scn_conv_tc_take_error(void);

/* Device address of that code word on the current device (NULL if it cannot be resolved), for
 * callers that would rather copy it with results they fetch anyway than wait in
 * scn_conv_tc_take_error.  A non-zero word read this way stays set until
 * scn_conv_tc_take_error or scn_classifier_result clears it.  No reference counterpart. */
const int *scn_conv_tc_error_word(void);

/* Replaces propForwardToMatrixMultiply alone (ConvolutionalLayer.cu:12-41): the
 * materialised gather, for callers that read ConvolutionalLayer's output themselves.
 * out[c*nIn + j] = in[rules[c]*nIn + j], zero where rules[c] < 0; count = rows_out*fs. */
int scn_gather_forward(const float *d_in, const int *d_rules, long long count, int nIn,
                       float *d_out, scn_stream_t stream);

/* d_bg[b] = the row of sample b whose key is negative (its background row, the value every
 * Picture::codifyInputData stores in SparseGrid::backgroundCol, e.g. OpenCVPicture.cpp:373-375),
 * or -1: lets a caller upload keys and offsets only. */
int scn_background_rows(const int *d_keys, const int *d_off, int batch, int *d_bg, scn_stream_t stream);

/* Replaces applySigmoid and PreLU as stand-alone passes (SigmoidLayer.cu:187-222;
 * NetworkInNetworkPReLULayer.cu:8-23): d_out = act(d_in) over [rows x N], in place allowed.
 * The layer kernels fuse their activation; this is for callers that apply one themselves. */
int scn_activation_forward(const float *d_in, float *d_out, int rows, int N, int act,
                           const float *d_prelu, scn_stream_t stream);

/* Replaces maxPool / dMaxPool (MaxPoolingLayer.cu:9-72): per output row and channel the
 * maximum over the row's non-negative rules, first maximum wins, and the flat input index
 * rule*C + channel of the winner in d_choices (SpatiallySparseBatchSubInterface::
 * poolingChoices).  Rows without a usable rule give 0 and -1. */
int scn_maxpool_forward(const float *d_in, const int *d_rules, int rows_out, int sd, int C,
                        float *d_out, int *d_choices, scn_stream_t stream);

/* Replaces terminalPool / dTerminalPool (TerminalPoolingLayer.cu:22-46): mean over each
 * row's rules up to the first negative one. */
int scn_terminal_pool_forward(const float *d_in, const int *d_rules, int batch, int S, int C,
                              float *d_out, scn_stream_t stream);

/* Replaces the device half of SoftmaxClassifier plus vectorTopIndices
 * (SoftmaxClassifier.cu:16-41; utilities.cu:35-56): per row of d_probs[rows x nClasses]
 * the nTop largest classes in descending order (ties: lowest index first) into
 * d_top[rows x nTop]. */
int scn_top_indices(const float *d_probs, int rows, int nClasses, int nTop, int *d_top,
                    scn_stream_t stream);

/* The same device half of SoftmaxClassifier (SoftmaxClassifier.cu:31-41: the copy of the
 * probabilities to the host and vectorTopIndices per row) with everything the host reads back
 * laid out as ONE block, so that one device-to-host copy fetches it:
 *   float probs[rows * nClasses]; int top[rows * nTop]; int tc_error;
 * tc_error is the code word of scn_conv_tc_take_error, taken (read and cleared) by this
 * kernel: non-zero means a tensor-core kernel before it gave up a wait and the probabilities
 * are not to be trusted.  scn_classifier_result_bytes gives the block's size. */
size_t scn_classifier_result_bytes(int rows, int nClasses, int nTop);
int scn_classifier_result(const float *d_probs, int rows, int nClasses, int nTop, void *d_block,
                          scn_stream_t stream);

/* ------------------------------------------------------------------ backward pass (training step)
 * The reference runs every layer's backwards() in reverse order behind SoftmaxClassifier
 * (SparseConvNetCUDA.cu:247-251).  Training-time dropout (random feature subsets and the
 * shrunk weight matrices, NetworkInNetworkLayer.cu:162-186) keeps full-width matrices here:
 * see scn_mask_columns and scn_sgd_update_masked below. */

/* Replaces dDerivativeOfCostWRTpreSoftmaxTopLevelWeights (SoftmaxClassifier.cu:7-14, 27-33):
 * d_dfeatures[r][c] = d_probs[r][c] - (c == d_labels[r]), not averaged over the batch. */
int scn_softmax_nll_backward(const float *d_probs, const int *d_labels, int rows, int nClasses,
                             float *d_dfeatures, scn_stream_t stream);

/* Replaces applySigmoidBackProp (SigmoidLayer.cu:224-268) and PReLUBackprop
 * (NetworkInNetworkPReLULayer.cu:25-47), in place on the output's gradient: d *= f'(.),
 * the derivative taken from the ACTIVATED features as the reference takes it.  PReLU also
 * gets the slope gradient d_dprelu[N] = sum over rows of d * (b > 0 ? 0 : b / slope).
 * Softmax and NOSIGMOID pass through. */
int scn_activation_backward(const float *d_out_features, float *d_dfeatures, int rows, int N, int act,
                            const float *d_prelu, float *d_dprelu, scn_stream_t stream);

/* Replaces the weight half of NetworkInNetworkLayer::backwards (NetworkInNetworkLayer.cu:226-239:
 * cuBLAS SGEMM X^T d, columnSum) with the convolution's gather read through the rulebook
 * inside the kernel (the gathered matrix is never written): d_dW[(fs*nIn) x N] = X^T d_dout,
 * d_dB[N] = column sums of d_dout; X as in scn_conv_nin_forward (d_rules NULL and fs 1: plain). */
int scn_conv_nin_backward_weights(const float *d_in, const int *d_rules, int rows, int fs, int nIn,
                                  const float *d_dout, int N, float *d_dW, float *d_dB, scn_stream_t stream);

/* The same weight gradient on the tensor cores (three tf32 products): the gathered input is written once, transposed,
 * the output gradient is packed like a weight matrix, and the fused forward kernel multiplies them with the roles
 * turned (its rows = the fs*nIn input channels, its contraction = the layer's rows), K split over the CTAs.
 * Workspace: scn_conv_nin_backward_weights_tc_bytes (0: shape not taken -- fewer than 128 rows, N below 16 or not a
 * multiple of 4 --, for which the call answers SCN_ERR_UNSUPPORTED: use scn_conv_nin_backward_weights). */
size_t scn_conv_nin_backward_weights_tc_bytes(int rows, int fs, int nIn, int N);
int scn_conv_nin_backward_weights_tc(const float *d_in, const int *d_rules, int rows, int fs, int nIn, const float *d_dout,
                                     int N, float *d_dW, float *d_dB, void *d_workspace, size_t workspace_bytes,
                                     scn_stream_t stream);

/* d_Wt[N x K] = transpose of d_W[K x N].  The input half of NetworkInNetworkLayer::backwards
 * (NetworkInNetworkLayer.cu:266-277: dX = d W^T) is scn_conv_nin_forward_ws on d_dout with
 * these transposed weights (zero bias, no activation), so it runs on the tensor cores
 * wherever the forward pass does. */
int scn_transpose_weights(const float *d_W, int K, int N, float *d_Wt, scn_stream_t stream);

/* Replaces propBackwardFromMatrixMultiply (ConvolutionalLayer.cu:42-72): zeroes
 * d_din[rows_in x nIn], then d_din[rules[c]] += d_dconv[c] for the count = rows_out*fs rule
 * cells with a non-negative rule.  rows_in = 0: nothing is zeroed (the reference's free function:
 * the caller has zeroed d_din). */
int scn_gather_backward(const float *d_dconv, const int *d_rules, long long count, int nIn, float *d_din,
                        long long rows_in, scn_stream_t stream);

/* Replaces maxPoolBackProp (MaxPoolingLayer.cu:74-93, 134-146): zeroes d_din[n_in], then
 * d_din[d_choices[i]] += d_dout[i] for the n pooled values.  n_in = 0: nothing is zeroed. */
int scn_maxpool_backward(const float *d_dout, const int *d_choices, long long n, float *d_din, long long n_in,
                         scn_stream_t stream);

/* Replaces terminalPoolBackProp (TerminalPoolingLayer.cu:48-73, 112-125): zeroes
 * d_din[rows_in x C]; every input row a sample pooled receives that sample's gradient
 * divided by the number of rows pooled. */
int scn_terminal_pool_backward(const float *d_dout, const int *d_rules, int batch, int S, int C, float *d_din,
                               long long rows_in, scn_stream_t stream);

/* Replaces dGradientDescent (NetworkInNetworkLayer.cu:26-40): w -= m*momentum;
 * m = momentum*m - learningRate*(1-momentum)*delta; w += m*(1+momentum); with keep_positive
 * also dGradientDescentKeepPositive (NetworkInNetworkPReLULayer.cu:67-84), the PReLU slopes'
 * update, which then holds w at 0.001 or above. */
int scn_sgd_update(float *d_w, float *d_momentum, const float *d_delta, long long n, float learningRate,
                   float momentum, int keep_positive, scn_stream_t stream);

/* Training-time dropout (NetworkInNetworkLayer.cu:152-186, 240-263) with full-width matrices: instead of shrinking W, the
 * features and the gradients to the features a batch keeps, the dropped features' columns are zeroed
 * (scn_mask_columns: d_x[r][n] = 0 where d_mask[n] == 0) and the update skips the weights of dropped input and output
 * features (scn_sgd_update_masked: entry (row, col) of d_w[rows x N] is updated like scn_sgd_update unless
 * d_row_mask[row % row_period] == 0 or d_col_mask[col] == 0; either mask may be NULL).  The values the reference's narrow
 * matrices hold are the same. */
int scn_mask_columns(float *d_x, long long rows, int N, const float *d_mask, scn_stream_t stream);
int scn_sgd_update_masked(float *d_w, float *d_momentum, const float *d_delta, long long rows, int N,
                          const float *d_row_mask, int row_period, const float *d_col_mask, float learningRate,
                          float momentum, int keep_positive, scn_stream_t stream);

/* Index learning (IndexLearnerLayer.cu:8-20, 57-66): d_w[k][j] = d_W[k][d_idx[j]] for the n columns of d_W [K x N] a batch
 * indexes, and d_W[k][d_idx[j]] += alpha * d_delta[k][j] (the update without momentum; the indices must be distinct). */
int scn_gather_columns(const float *d_W, int K, int N, const int *d_idx, int n, float *d_w, scn_stream_t stream);
int scn_scatter_columns_axpy(float *d_W, int K, int N, const int *d_idx, int n, const float *d_delta, float alpha,
                             scn_stream_t stream);

/* The reference's four cuBLAS wrappers (utilities.cu:132-169) as one call: C[l x r] = alpha * op(A) * op(B) + beta * C on
 * row-major fp32 matrices, op(A) l x m, op(B) m x r; transA / transB non-zero: that operand is stored transposed (m x l,
 * r x m).  CUDA cores; not used by the forward path. */
int scn_sgemm_rowmajor(int transA, int transB, const float *d_A, const float *d_B, float *d_C, int l, int m, int r,
                       float alpha, float beta, scn_stream_t stream);

/* ------------------------------------------------------------------ result exchange between the GPUs of one node
 * The reference runs on one GPU (SparseConvNetCUDA.cu:43-71 picks a single device).  Sharded by sample over several
 * GPUs, the path has one exchange step: every rank's [rows x nClasses] block of probabilities (what
 * SoftmaxClassifier.cu:36-41 copies to the host) goes to every other rank.  These calls do that over peer memory, on
 * the rank's own stream, without a host-side collective:
 *   scn_exchange_buffer_bytes   size of a rank's buffer for `world` ranks (at most 16) and blocks of at most
 *                               cap_floats floats (0 = bad arguments);
 *   scn_exchange_alloc          cudaMalloc + clear such a buffer and, where ipc_handle is not NULL, write the 64 bytes
 *                               another process of this node passes to scn_exchange_open to map it;
 *   scn_exchange_publish        store d_block[floats] (rows = its row count, carried along) into the buffer of every rank
 *                               named in peers[world] (host array of device pointers, own buffer included) and
 *                               announce it as `step` (1, 2, 3, ... on every rank alike);
 *   scn_exchange_collect        wait until every rank's block of `step` has arrived in d_local, then
 *                               d_out[r * cap_floats ...] = rank r's block and d_rows[r] = its row count (d_rows may be
 *                               NULL).  A rank whose block does not arrive within the time limit
 *                               (scn_exchange_set_timeout_ms, 2000 by default) gets bit r of *d_status set and its part
 *                               of d_out left as it was; the kernel always returns.
 *   scn_exchange_step           both in ONE launch: collect `collect_step` (0 = nothing to collect), publish
 *                               `publish_step` (0 = nothing to publish), collect_step < publish_step.
 * A rank must collect step s before it publishes step s + 1; with that order four slots per source are enough for
 * a slot never to be overwritten before its owner has read it. */
size_t scn_exchange_buffer_bytes(int world, int cap_floats);
void scn_exchange_set_timeout_ms(int ms);
int scn_exchange_alloc(size_t bytes, void **d_buffer, unsigned char *ipc_handle);
int scn_exchange_free(void *d_buffer);
int scn_exchange_open(const unsigned char *ipc_handle, void **d_peer);
int scn_exchange_close(void *d_peer);
int scn_exchange_publish(const float *d_block, int floats, int rows, void *const *peers, int world, int rank, int cap_floats,
                         unsigned step, scn_stream_t stream);
int scn_exchange_collect(void *d_local, int world, int cap_floats, unsigned step, float *d_out, int *d_rows, int *d_status,
                         scn_stream_t stream);
int scn_exchange_step(void *d_local, unsigned collect_step, float *d_out, int *d_rows, int *d_status, const float *d_block, int floats,
                      int rows, void *const *peers, int world, int rank, int cap_floats, unsigned publish_step, scn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SCN_B200_H */
