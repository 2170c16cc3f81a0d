/* scn_b200_net -- C entry points of libscn_b200_host.so, the C++ host library whose classes
 * keep the reference's names (SparseConvNetCUDA, the layer classes, vectorCUDA,
 * SpatiallySparseBatchInterface, NetworkArchitectures; headers under
 * sparseconvnet-archived_b200/csrc/host/).  C++ callers use those classes directly; this
 * header exists for hosts that cannot (the Python test and benchmark harness binds it with
 * ctypes).  Each function wraps the reference-named method given in its comment (paths
 * inside the reference project, SparseConvNet/...).
 *
 * All functions return 0 on success, non-zero on failure with scn_net_last_error() set;
 * nothing prints an error or exits.  Buffers named h_* are host memory, d_* device memory.
 */
#ifndef SCN_B200_NET_H
#define SCN_B200_NET_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct scn_net scn_net_t;

const char *scn_net_last_error(void);

/* SparseConvNetCUDA::SparseConvNetCUDA (SparseConvNetCUDA.cu:24-42).  `stream` is a
 * cudaStream_t to enqueue on, or NULL for a stream of the network's own; the current CUDA
 * device is used.  lattice: 0 square/cubic (SparseConvNet), 1 triangular/tetrahedral
 * (SparseConvTriangLeNet). */
scn_net_t *scn_net_create(int dimension, int nInputFeatures, int nClasses, int nTop, int lattice, void *stream);
void scn_net_destroy(scn_net_t *net);

/* SparseConvNet::addLeNetLayerMP / SparseConvTriangLeNet::addLeNetLayerMP (SparseConvNet.h:29-32, 80-83). */
int scn_net_addLeNetLayerMP(scn_net_t *net, int nFeatures, int filterSize, int filterStride, int poolSize, int poolStride,
                            int activationFn, float dropout, int minActiveInputs);
/* SparseConvNet::addTerminalPoolingLayer (SparseConvNet.cu:56-58, 123-126). */
/* SparseConvNet::addLeNetLayer{PO,PD,RO,RD}FMP (SparseConvNet.h:32-47): kind 0 pseudorandom overlapping,
 * 1 pseudorandom non-overlapping, 2 random overlapping, 3 random non-overlapping. */
int scn_net_addLeNetLayerFMP(scn_net_t *net, int kind, int nFeatures, int filterSize, int filterStride, int poolSize,
                             float fmpShrink, int activation, float dropout, int minActiveInputs);
/* Turns the fusion of convolution + learnt layer + non-overlapping max pooling into one kernel on (the
 * builders' default) or off; off, every learnt layer writes its output, as the reference does. */
int scn_net_set_pool_fusion(scn_net_t *net, int on);
/* Re-seeds the RNG of every fractional max-pooling layer (layer index l gets seed + l) so that the next
 * forward draws a known sequence of region bounds.  The reference seeds from the clock (Rng.cpp:8-15). */
int scn_net_seed_fmp(scn_net_t *net, unsigned seed);
int scn_net_addTerminalPoolingLayer(scn_net_t *net, int poolSize);
/* SparseConvNetCUDA::addSoftmaxLayer (SparseConvNetCUDA.cu:200-213). */
int scn_net_addSoftmaxLayer(scn_net_t *net);
/* DeepCNet::DeepCNet (NetworkArchitectures.cpp:3-11), on the given stream. */
scn_net_t *scn_net_DeepCNet(int dimension, int l, int k, int fn, int nInputFeatures, int nClasses, float p, int nTop, void *stream);
/* Any of the named architectures (NetworkArchitectures.h:4-69), built by constructing the class of that name
 * on the default device: DeepCNet DeepC2 DeepCNiN DeepC2C2 DeepC3C3Valid DeepC3C3 POFMPSparseConvNet
 * ROFMPSparseConvNet PDFMPSparseConvNet RDFMPSparseConvNet.  fmpShrink is read by the last four only.
 * NULL (and scn_net_last_error) for an unknown name or a builder that refuses its arguments. */
scn_net_t *scn_net_named(const char *name, int dimension, int l, int k, float fmpShrink, int fn, int nInputFeatures, int nClasses, float p,
                         int nTop);

int scn_net_n_layers(scn_net_t *net);
int scn_net_input_spatial_size(scn_net_t *net);
/* info[10] = type (0 conv, 1 triangular conv, 2 NiN, 3 max pool, 4 triangular max pool,
 * 5 terminal pool), size, stride, minActiveInputs, nFeaturesIn, nFeaturesOut, cells,
 * activation, inSpatialSize, outSpatialSize.  For a max pooling layer `activation` is 1 when its last
 * forward ran inside the kernel of the convolution + learnt layer in front of it, else 0. */
int scn_net_layer_info(scn_net_t *net, int layer, int *info, float *dropout);
/* Set NetworkInNetworkLayer::W, B (and PReLU) of layer `layer` from host arrays
 * (NetworkInNetworkLayer.h:12-19). */
int scn_net_set_weights(scn_net_t *net, int layer, const float *h_W, const float *h_B, const float *h_prelu);
/* SparseConvNetCUDA::loadWeights / saveWeights (SparseConvNetCUDA.cu:406-442), momentum = false. */
int scn_net_load_weights(scn_net_t *net, const char *baseName, int epoch);
int scn_net_save_weights(scn_net_t *net, const char *baseName, int epoch);
/* scn_precision for every NetworkInNetwork layer (default SCN_PREC_AUTO).  A tensor-core precision
 * applies to the layers whose shape has a tensor-core path (N >= 16, N % 4 == 0); the others (the
 * classifier, say) keep the fp32 CUDA-core kernel. */
int scn_net_set_precision(scn_net_t *net, int precision);

/* One batch end to end from HOST buffers, as BatchProducer::nextBatch + processBatch do
 * (BatchProducer.cu:108-142; SparseConvNetCUDA.cu:227-271): upload, rule chain on the
 * device, all layers, classifier read-back.
 *   h_keys[rows]  site key per row, -1 for a sample's background row
 *   h_off[batch+1] first row of each sample;  h_features[rows x nInputFeatures]
 *   h_probs[batch x nClasses], h_predictions[batch x nTop] (either may be NULL) */
int scn_net_forward_host(scn_net_t *net, int batch, const int *h_keys, const int *h_off, const float *h_features,
                         float *h_probs, int *h_predictions);
/* One training step on one batch given like scn_net_forward_host plus one label per sample:
 * the TRAINBATCH branch of SparseConvNetCUDA::processBatch (SparseConvNetCUDA.cu:227-251):
 * forward, SoftmaxClassifier (negative log-likelihood and mistakes into stats[0..1], the
 * probabilities into h_probs), every layer's backwards() in reverse order with the SGD update
 * of its weights (learningRate, momentum as in NetworkInNetworkLayer.cu:26-40).  The samples
 * stay in the order given.  A learnt layer with dropout d keeps floor(nOut (1 - d)) randomly drawn output features per
 * batch (NetworkInNetworkLayer.cu:152-154): the others are zero in the forward pass and untouched by the update. */
int scn_net_train_batch(scn_net_t *net, int batch, const int *h_keys, const int *h_off, const float *h_features, const int *h_labels,
                        float learningRate, float momentum, float *h_probs, double *stats);
/* The output features learnt layer `layer` keeps in the training batches that follow, instead of a random draw: n
 * ascending indices below its nFeaturesOut (n = 0: back to random draws).  For repeating a run with known subsets. */
int scn_net_set_dropout_features(scn_net_t *net, int layer, const int *present, int n);
/* The features interface i kept in the last batch (see above): returns their count, which is the interface's nFeatures
 * unless it is a learnt layer's output in a training batch with dropout, and copies the indices if `present` is not NULL. */
int scn_net_iface_present(scn_net_t *net, int i, int *present);
/* Index learning (IndexLearnerLayer.h, SparseConvNetCUDA.cu:211-225, 443-474): addIndexLearnerLayer in place of
 * addSoftmaxLayer makes nClasses the number of pictures of the training set; a step runs every layer, the index learner on
 * the columns `sample_numbers` (each picture's number in the training set, distinct), IndexLearner (picture i's class is
 * column i: h_probs [batch x batch], stats = {negative log-likelihood, mistakes}) and the backward pass (the index learner
 * updates without momentum). */
int scn_net_addIndexLearnerLayer(scn_net_t *net);
int scn_net_index_learner_batch(scn_net_t *net, int batch, const int *h_keys, const int *h_off, const float *h_features,
                                const int *sample_numbers, float learningRate, float momentum, float *h_probs, double *stats);
/* One RESCALEBATCH through processBatch (SparseConvNetCUDA.cu:230-240): every layer's forwards followed by its
 * scaleWeights (NetworkInNetworkLayer.cu:203-220: weights and biases scaled by the -0.1th power of the layer's mean
 * absolute output, the scale applied underneath divided out again, the top layer left alone). */
int scn_net_rescale_batch(scn_net_t *net, int batch, const int *keys, const int *off, const float *features);
/* A learnt layer's weights as they are now (W [nIn x nOut], B [nOut], PReLU slopes [nOut] or NULL). */
int scn_net_get_weights(scn_net_t *net, int layer, float *h_W, float *h_B, float *h_prelu);
/* d cost / d features of interface i after scn_net_train_batch: returns their count (-1 on
 * error, 0 where no gradient reaches) and copies them when h_dfeatures is not NULL. */
long long scn_net_iface_dfeatures(scn_net_t *net, int i, float *h_dfeatures);

/* The same with inputs already resident in device memory: the batch's interface reads the caller's
 * arrays in place (no copy), so they must stay unchanged until the forward has run on the stream and
 * must not be freed before the network's next forward call.  d_bg[batch] is each sample's background row or -1;
 * maxSitesPerSample the largest site count of a sample.  Results are left on the device:
 * d_probs[batch x nClasses], d_top[batch x nTop] (either may be NULL).  Does not wait for
 * the stream beyond the rule chain's one read-back. */
int scn_net_forward_device(scn_net_t *net, int batch, int rows, int maxSitesPerSample, const int *d_keys, const int *d_off,
                           const int *d_bg, const float *d_features, float *d_probs, int *d_top);

/* Copy the class probabilities of the last forward (the top interface's features,
 * [batch x nClasses]) to d_probs on the network's stream, e.g. into an all-gather buffer. */
int scn_net_copy_probs_device(scn_net_t *net, float *d_probs);

/* SpatiallySparseBatchInterface i of the last forward (0 = input, i+1 = output of layer i;
 * SpatiallySparseBatchInterface.h:19-46).  sizes[5] = nSpatialSites, nFeatures, spatialSize,
 * rules.size(), poolingChoices.size() (0 unless layer i-1 pools).  A ConvolutionalLayer
 * fused into the next layer has no materialised features: its nFeatures is reported but
 * fetching its features fails unless h_features is NULL. */
int scn_net_iface_sizes(scn_net_t *net, int i, long long *sizes);
int scn_net_iface_fetch(scn_net_t *net, int i, float *h_features, int *h_rules, int *h_choices, int *h_rowKeys);

/* multiplyAddCount since the last call (types.h:46-52; NetworkInNetworkLayer.cu:197-199). */
double scn_net_take_multiply_adds(void);

/* CUDA-event timing of each layer's forwards() and of the rule chain, for roofline reports.
 * After a forward and a stream synchronisation, h_ms[0..n_layers) holds the milliseconds of
 * each layer's forward kernels and h_ms[n_layers] the rule chain (uploads excluded). */
int scn_net_enable_timing(scn_net_t *net, int on);
int scn_net_layer_times(scn_net_t *net, float *h_ms);

/* Run a small synthetic dataset of SitesPicture objects through
 * SparseConvNetCUDA::processDataset with its BatchProducer threads
 * (SparseConvNetCUDA.cu:272-326; BatchProducer.cu): same flat input as
 * scn_net_forward_host plus labels; returns the error rate through *errorRate and the
 * per-sample probabilities of the pass in h_probs. */
int scn_net_process_dataset(scn_net_t *net, int nSamples, const int *h_keys, const int *h_off, const float *h_features,
                            const int *h_labels, int batchSize, float *errorRate, float *h_probs);

/* vectorTopIndices (utilities.cu:35-56), the host version SoftmaxClassifier-style callers use. */
int scn_host_vectorTopIndices(const float *h_v, int n, int k, int *h_out);

/* scn_net_forward_host in two halves, so that a caller with a stream of batches overlaps the upload of the next
 * batch with the computation of the current one, as the reference's producer threads do for its consumer thread
 * (BatchProducer.cu:90-142, SparseConvNetCUDA.cu:272-326): _begin starts the copies of a batch's host arrays (which
 * must stay as they are until the matching _end returns; page-locked memory makes the copies asynchronous) and
 * returns; _end computes the oldest batch begun and not yet ended and returns its results.  At most two batches may be
 * on their way.  With gathered_prev / rows_prev not NULL, _end also does what scn_net_forward_host_exchange does. */
int scn_net_forward_host_begin(scn_net_t *net, int batch, const int *keys, const int *off, const float *features);
int scn_net_forward_host_end(scn_net_t *net, float *probs, int *predictions, float *gathered_prev, int *rows_prev);

/* ---- results of a batch sharded by sample over the GPUs of one node (ResultExchange: peer stores + bounded waits,
 * no host-side collective; the reference itself runs on one device, SparseConvNetCUDA.cu:43-71).
 * scn_net_exchange_create allocates this rank's buffer for blocks of at most cap_rows x nClasses probabilities and
 * writes the 64 bytes (handle_out) that the other ranks' processes need; scn_net_exchange_connect takes all ranks'
 * 64-byte entries in rank order (world x 64 bytes; how they travel is the caller's business: one all-gather at
 * start-up).  Ranks that live in ONE process (tests) pass each other's scn_net_exchange_buffer pointers to
 * scn_net_exchange_connect_local instead.  Every rank must run the same sequence of exchange steps.  Before
 * scn_net_exchange_destroy / scn_net_destroy the ranks synchronise (no peer may still be storing into the buffer). */
int scn_net_exchange_create(scn_net_t *net, int world, int rank, int cap_rows, unsigned char *handle_out);
void *scn_net_exchange_buffer(scn_net_t *net);
int scn_net_exchange_connect(scn_net_t *net, const unsigned char *handles);
int scn_net_exchange_connect_local(scn_net_t *net, void *const *buffers);
int scn_net_exchange_destroy(scn_net_t *net);
/* scn_net_forward_host that also publishes this step's probabilities to every rank and returns what every rank
 * published in the step BEFORE: gathered_prev[world x cap_rows x nClasses] (rank r's block at r * cap_rows * nClasses)
 * and rows_prev[world] (-1 everywhere on the first step).  One copy-and-wait ends the step, as in scn_net_forward_host.
 * A rank whose block has not arrived within the time limit (scn_exchange_set_timeout_ms) makes the call fail. */
int scn_net_forward_host_exchange(scn_net_t *net, int batch, const int *keys, const int *off, const float *features, float *probs,
                                  int *predictions, float *gathered_prev, int *rows_prev);
/* The blocks of the last published step (ends a run of scn_net_forward_host_exchange calls; waits for the stream). */
int scn_net_exchange_flush(scn_net_t *net, float *gathered, int *rows);
/* Device-resident form, enqueued without waiting: collects the step before into
 * d_gathered_prev[world x cap_rows x nClasses] and d_rows_status_prev[world + 1] (row counts, then a word with bit r
 * set if rank r's block did not arrive in time), then publishes d_probs[rows x nClasses] as the next step
 * (d_probs NULL: collect only).  The kernel runs on a stream of the exchange's own, ordered behind what the network's
 * stream holds at the call, so the next forward does not queue behind it: d_probs must stay as it is, and what was
 * collected is complete, for work enqueued on the network's stream after the NEXT call (after this one when d_probs
 * is NULL, which is how a run of steps ends).  A host-buffer step (scn_net_forward_host_exchange) must not follow
 * before such a collect-only call. */
int scn_net_exchange_step_device(scn_net_t *net, const float *d_probs, int rows, float *d_gathered_prev, int *d_rows_status_prev);

#ifdef __cplusplus
}
#endif
#endif
