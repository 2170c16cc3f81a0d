"""TEST INFRASTRUCTURE ONLY: ctypes bindings for the parity oracle.

`Oracle` wraps oracle/_build/libscn_oracle.so (the CPU restatement, scn_oracle.cpp) and
`Reference` wraps oracle/_ref/libscn_ref.so (the reference's own Regions.cu compiled
unchanged, see the Makefile) and `ReferenceGPU` wraps oracle/_ref_gpu/libscn_ref_gpu.so (the
reference's own network classes and CUDA kernels compiled unchanged for the GPU; it needs a
CUDA device and is used by GPU tests only).  Only tests/, the smoke check and the benchmark's CPU-baseline
legs import this module; the product package never does.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libscn_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libscn_ref.so")
REF_GPU_SO = os.path.join(HERE, "_ref_gpu", "libscn_ref_gpu.so")

c_int, c_ll, c_f, c_p, c_d = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p, ctypes.c_double

# ActivationFunction (types.h:20-29)
NOSIGMOID, RELU, VLEAKYRELU, LEAKYRELU, TANH, SOFTMAX, PRELU, SIGMOID = range(8)
# layer types of scn_oracle.cpp
L_CONV, L_CONV_TRI, L_NIN, L_MAXPOOL, L_MAXPOOL_TRI, L_TERMINAL = range(6)
# fractional max-pooling tick kinds: pseudorandom/random x overlapping/non-overlapping ("disjoint")
FMP_PO, FMP_PD, FMP_RO, FMP_RD = range(4)


# where the reference checkout lies on the machine that builds oracle/_ref and oracle/_ref_gpu: named by
# SCN_REFERENCE_DIR, else looked for beside this repository
REF_DIR = os.environ.get("SCN_REFERENCE_DIR") or os.path.normpath(os.path.join(HERE, "..", "..", "reference", "SparseConvNet"))


def build(force=False):
    """Compile the oracle (and oracle/_ref when the reference checkout is present)."""
    if force or not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(
            os.path.join(HERE, "scn_oracle.cpp")):
        subprocess.check_call(["make", "-C", HERE, "oracle"], stdout=subprocess.DEVNULL)
    if os.path.isdir(REF_DIR) and (force or not os.path.exists(REF_SO) or os.path.getmtime(REF_SO) < os.path.getmtime(
            os.path.join(HERE, "ref_wrap.cpp"))):
        subprocess.check_call(["make", "-C", HERE, "_ref", "REF=" + REF_DIR], stdout=subprocess.DEVNULL)
    if os.path.isdir(REF_DIR) and (force or not os.path.exists(REF_GPU_SO) or os.path.getmtime(REF_GPU_SO) < os.path.getmtime(
            os.path.join(HERE, "ref_gpu_wrap.cu"))):
        subprocess.check_call(["make", "-C", HERE, "_ref_gpu", "REF=" + REF_DIR], stdout=subprocess.DEVNULL)


def _p(a):
    return None if a is None else a.ctypes.data_as(c_p)


class _RulesLib:
    """Shared flat protocol of orc_grid_rules / ref_grid_rules."""

    def __init__(self, path, prefix):
        self.lib = ctypes.CDLL(path)
        L, self.pre = self.lib, prefix
        f = getattr(L, prefix + "_grid_rules")
        f.restype, f.argtypes = c_p, [c_int] * 8 + [c_p] * 4
        for n in ("n_rules", "n_out"):
            g = getattr(L, prefix + "_result_" + n)
            g.restype, g.argtypes = c_ll, [c_p]
        g = getattr(L, prefix + "_result_n_sites")
        g.restype, g.argtypes = c_int, [c_p]
        getattr(L, prefix + "_result_fetch").argtypes = [c_p] * 6
        getattr(L, prefix + "_result_free").argtypes = [c_p]

    def grid_rules(self, kind, dim, nIn, nOut, size, stride, minActive, keys, rows, off, bg):
        """-> dict(rules, out_keys, out_rows, out_off, out_bg, n_sites); one call = one layer's
        preprocess over a batch (row ids run on across samples)."""
        keys = np.ascontiguousarray(keys, np.int64)
        rows = np.ascontiguousarray(rows, np.int32)
        off = np.ascontiguousarray(off, np.int32)
        bg = np.ascontiguousarray(bg, np.int32)
        B = len(bg)
        L, pre = self.lib, self.pre
        h = getattr(L, pre + "_grid_rules")(kind, dim, nIn, nOut, size, stride, minActive, B,
                                            _p(keys), _p(rows), _p(off), _p(bg))
        return self._fetch(h, B)

    def _fetch(self, h, B):
        L, pre = self.lib, self.pre
        nr = getattr(L, pre + "_result_n_rules")(h)
        no = getattr(L, pre + "_result_n_out")(h)
        ns = getattr(L, pre + "_result_n_sites")(h)
        rules = np.zeros(nr, np.int32)
        ok, orow = np.zeros(no, np.int64), np.zeros(no, np.int32)
        ooff, obg = np.zeros(B + 1, np.int32), np.zeros(B, np.int32)
        getattr(L, pre + "_result_fetch")(h, _p(rules), _p(ok), _p(orow), _p(ooff), _p(obg))
        getattr(L, pre + "_result_free")(h)
        return dict(rules=rules, out_keys=ok, out_rows=orow, out_off=ooff, out_bg=obg, n_sites=ns)


class Reference(_RulesLib):
    """The reference's own rule construction (vectorHash order)."""

    def __init__(self):
        super().__init__(REF_SO, "ref")
        L = self.lib
        for n in ("ref_ipow", "ref_triangleSize", "ref_intRound"):
            getattr(L, n).restype, getattr(L, n).argtypes = c_int, [c_int, c_int]
        L.ref_vectorTopIndices.argtypes = [c_p, c_int, c_int, c_p]

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def top_indices(self, v, k):
        v = np.ascontiguousarray(v, np.float32)
        out = np.zeros(k, np.int32)
        self.lib.ref_vectorTopIndices(_p(v), len(v), k, _p(out))
        return out

    def fmp_rules(self, kind, dim, nIn, nOut, poolSize, seed, keys, rows, off, bg):
        """One fractional max-pooling layer's preprocess over a batch with the layer RNG re-seeded
        (kind: FMP_PO, FMP_PD, FMP_RO, FMP_RD) -> (result dict, ticks[batch, dim, 2*nOut + 2*nIn])."""
        keys, rows = np.ascontiguousarray(keys, np.int64), np.ascontiguousarray(rows, np.int32)
        off, bg = np.ascontiguousarray(off, np.int32), np.ascontiguousarray(bg, np.int32)
        B = len(bg)
        ticks = np.zeros((B, dim, 2 * nOut + 2 * nIn), np.int32)
        f = self.lib.ref_fmp_rules
        f.restype, f.argtypes = c_p, [c_int] * 5 + [ctypes.c_uint, c_int] + [c_p] * 5
        h = f(kind, dim, nIn, nOut, poolSize, seed, B, _p(keys), _p(rows), _p(off), _p(bg), _p(ticks))
        return self._fetch(h, B), ticks


class ReferenceGPU:
    """The reference's own SparseConvNetCUDA (builders, BatchProducer, layer classes, CUDA kernels, cuBLAS
    SGEMM) on the current CUDA device, one batch at a time.  Mirrors OracleNet's builder calls."""

    def __init__(self, dim, nInputFeatures, nClasses, nTop=1, lattice=0, named=None):
        """named = (name, l, k, fn, p, fmpShrink): construct the reference's class of that name
        (NetworkArchitectures.cpp) instead of an empty network."""
        self.L = L = ctypes.CDLL(REF_GPU_SO)
        L.refgpu_create.restype, L.refgpu_create.argtypes = c_p, [c_int] * 5
        L.refgpu_named.restype = c_p
        L.refgpu_named.argtypes = [ctypes.c_char_p, c_int, c_int, c_int, c_f, c_int, c_int, c_int, c_f, c_int]
        L.refgpu_seed_fmp.argtypes = [c_p, ctypes.c_uint]
        L.refgpu_seed_dropout.argtypes = [c_p, ctypes.c_uint]
        L.refgpu_addIndexLearnerLayer.argtypes = [c_p]
        L.refgpu_index_learner_batch.restype, L.refgpu_index_learner_batch.argtypes = c_int, [c_p, c_int, c_p, c_p, c_p, c_int, c_f, c_f]
        L.refgpu_results_wide.argtypes = [c_p, c_int, c_p, c_p]
        L.refgpu_layer_describe.argtypes = [c_p, c_int, c_p]
        L.refgpu_destroy.argtypes = [c_p]
        L.refgpu_addLeNetLayerMP.argtypes = [c_p] + [c_int] * 6 + [c_f, c_int]
        L.refgpu_addTerminalPoolingLayer.argtypes = [c_p, c_int, c_int]
        L.refgpu_addSoftmaxLayer.argtypes = [c_p]
        L.refgpu_n_layers.restype, L.refgpu_n_layers.argtypes = c_int, [c_p]
        L.refgpu_input_spatial_size.restype, L.refgpu_input_spatial_size.argtypes = c_int, [c_p]
        L.refgpu_layer_info.argtypes = [c_p, c_int, c_p, c_p]
        L.refgpu_load_weights.argtypes = [c_p, ctypes.c_char_p, c_int]
        L.refgpu_save_weights.argtypes = [c_p, ctypes.c_char_p, c_int]
        L.refgpu_forward.restype, L.refgpu_forward.argtypes = c_int, [c_p, c_int, c_p, c_p, c_p, c_p, c_int, c_f, c_f]
        L.refgpu_multiply_adds.restype = c_d
        L.refgpu_last_cuda_error.restype = c_int
        L.refgpu_iface_sizes.argtypes = [c_p, c_int, c_p]
        L.refgpu_iface_fetch.argtypes = [c_p, c_int] + [c_p] * 6
        L.refgpu_iface_features_present.argtypes = [c_p, c_int, c_p]
        L.refgpu_results.argtypes = [c_p] * 4
        L.refgpu_layer_weights.argtypes = [c_p, c_int, c_p, c_p, c_p]
        L.refgpu_sample_numbers.argtypes = [c_p, c_p]
        self.dim, self.nIn, self.nClasses, self.nTop, self.lattice = dim, nInputFeatures, nClasses, nTop, lattice
        if named is None:
            self.h = L.refgpu_create(dim, nInputFeatures, nClasses, nTop, lattice)
        else:
            name, l, k, fn, p, fmpShrink = named
            self.h = L.refgpu_named(name.encode(), dim, l, k, fmpShrink, fn, nInputFeatures, nClasses, p, nTop)
            if not self.h:
                raise ValueError("unknown architecture " + name)

    def seed_fmp(self, seed):
        """Fractional max-pooling layer l draws from a generator seeded with seed + l from now on."""
        self.L.refgpu_seed_fmp(self.h, seed)

    def seed_dropout(self, seed):
        """Seed every learnt layer's dropout generator (seed + layer index): the subsets TRAINBATCHes draw then repeat."""
        self.L.refgpu_seed_dropout(self.h, seed)

    def describe(self):
        """Per layer the ten ints {type, size, stride, minActive, nIn, nOut, multiplier, fn, inSize, outSize}."""
        out = np.zeros((self.L.refgpu_n_layers(self.h), 10), np.int32)
        for i in range(out.shape[0]):
            self.L.refgpu_layer_describe(self.h, i, out[i].ctypes.data)
        return out

    @staticmethod
    def available():
        return os.path.exists(REF_GPU_SO)

    def __del__(self):
        try:
            self.L.refgpu_destroy(self.h)
        except Exception:
            pass

    def addLeNetLayerMP(self, nFeatures, fs, fstride, ps, pstride, act=RELU, dropout=0.0, minActive=1):
        self.L.refgpu_addLeNetLayerMP(self.h, nFeatures, fs, fstride, ps, pstride, act, dropout, minActive)

    def addTerminalPoolingLayer(self, poolSize, S=None):
        if S is None:  # the facades pass ipow / triangleSize (SparseConvNet.cu:56-58, 123-126)
            S = poolSize ** self.dim
            if self.lattice == 1:
                S = 1
                for k in range(self.dim):  # binomial(poolSize + dim - 1, dim)
                    S = S * (poolSize + k) // (k + 1)
        self.L.refgpu_addTerminalPoolingLayer(self.h, poolSize, S)

    def addSoftmaxLayer(self):
        self.L.refgpu_addSoftmaxLayer(self.h)

    def addIndexLearnerLayer(self):
        self.L.refgpu_addIndexLearnerLayer(self.h)

    def index_learner_batch(self, keys, off, features, batch_size, learning_rate, momentum):
        """One index-learning step of the reference on the first batch its BatchProducer draws from the pictures given.
        -> (sample numbers of the batch, probabilities [batch x batch], dict(nll, mistakes))."""
        keys = np.ascontiguousarray(keys, np.int64)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        n = self.L.refgpu_index_learner_batch(self.h, len(off) - 1, _p(keys), _p(off), _p(features), batch_size, learning_rate, momentum)
        err = self.L.refgpu_last_cuda_error()
        if n < 1 or err != 0:
            raise RuntimeError("reference index-learning step failed (%d pictures, CUDA error %d)" % (n, err))
        probs = np.zeros((n, n), np.float32)
        stats = np.zeros(2, np.float64)
        self.L.refgpu_results_wide(self.h, n, _p(probs), _p(stats))
        return self.sample_numbers(n), probs, dict(nll=float(stats[0]), mistakes=int(stats[1]))

    @property
    def inputSpatialSize(self):
        return self.L.refgpu_input_spatial_size(self.h)

    def layers(self):
        """Learnt-layer facts only: dict(learnt, nIn, nOut, act, dropout) per layer."""
        out = []
        for i in range(self.L.refgpu_n_layers(self.h)):
            info = np.zeros(5, np.int32)
            d = c_f()
            self.L.refgpu_layer_info(self.h, i, _p(info), ctypes.byref(d))
            out.append(dict(learnt=bool(info[0]), nIn=int(info[1]), nOut=int(info[2]), act=int(info[3]), dropout=float(d.value)))
        return out

    def load_weights(self, base, epoch):
        self.L.refgpu_load_weights(self.h, base.encode(), epoch)

    def save_weights(self, base, epoch):
        self.L.refgpu_save_weights(self.h, base.encode(), epoch)

    def forward(self, keys, off, features, labels=None, batch_type=2, learning_rate=0.0, momentum=0.0):
        """One batch through BatchProducer + processBatch.  batch_type 0 TRAINBATCH (also runs backwards and the SGD
        update), 1 TESTBATCH, 2 UNLABELEDBATCH.  -> (probabilities, predictions, dict(nll, mistakes, multiply_adds))."""
        keys = np.ascontiguousarray(keys, np.int64)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        labels = None if labels is None else np.ascontiguousarray(labels, np.int32)
        B = len(off) - 1
        n = self.L.refgpu_forward(self.h, B, _p(keys), _p(off), _p(features), _p(labels), batch_type, learning_rate, momentum)
        err = self.L.refgpu_last_cuda_error()
        if n != B or err != 0:
            raise RuntimeError("reference forward failed (processed %d of %d samples, CUDA error %d)" % (n, B, err))
        probs = np.zeros((B, self.nClasses), np.float32)
        pred = np.zeros((B, self.nTop), np.int32)
        stats = np.zeros(2, np.float64)
        self.L.refgpu_results(self.h, _p(probs), _p(pred), _p(stats))
        return probs, pred, dict(nll=float(stats[0]), mistakes=int(stats[1]), multiply_adds=float(self.L.refgpu_multiply_adds()))

    def iface(self, i):
        """Interface i of the last forward: 0 is the input, i+1 layer i's output."""
        s = np.zeros(8, np.int64)
        self.L.refgpu_iface_sizes(self.h, i, _p(s))
        rows, nF, sp, nr, nfp, nfeat, ndf, nch = (int(v) for v in s)
        feat, dfeat = np.zeros(nfeat, np.float32), np.zeros(ndf, np.float32)
        ch, rules = np.zeros(nch, np.int32), np.zeros(nr, np.int32)
        rk = np.zeros(rows, np.int64)
        self.L.refgpu_iface_fetch(self.h, i, _p(feat), _p(dfeat), _p(ch), _p(rules), _p(rk), None)
        w = nfp if nfp else nF
        present = np.zeros(nfp, np.int32)
        if nfp:
            self.L.refgpu_iface_features_present(self.h, i, _p(present))
        return dict(nSpatialSites=rows, nFeatures=nF, spatialSize=sp, featuresPresent=nfp, present=present,
                    features=feat.reshape(-1, w) if nfeat == rows * w else feat,
                    dfeatures=dfeat.reshape(-1, w) if ndf == rows * w else dfeat,
                    choices=ch, rules=rules, row_keys=rk)

    def sample_numbers(self, batch):
        """Position -> caller's sample index within the last batch (a TRAINBATCH is shuffled by the reference)."""
        out = np.zeros(batch, np.int32)
        self.L.refgpu_sample_numbers(self.h, _p(out))
        return out

    def layer_weights(self, i):
        info = self.layers()[i]
        W = np.zeros((info["nIn"], info["nOut"]), np.float32)
        B = np.zeros(info["nOut"], np.float32)
        pr = np.zeros(info["nOut"], np.float32)
        self.L.refgpu_layer_weights(self.h, i, _p(W), _p(B), _p(pr))
        return W, B, (pr if info["act"] == PRELU else None)


class Oracle(_RulesLib):
    def __init__(self):
        build()
        super().__init__(ORACLE_SO, "orc")
        L = self.lib
        for n in ("orc_ipow", "orc_triangleSize", "orc_intRound"):
            getattr(L, n).restype, getattr(L, n).argtypes = c_int, [c_int, c_int]
        L.orc_gather.argtypes = [c_p, c_p, c_ll, c_int, c_p]
        L.orc_nin_forward.argtypes = [c_p, c_ll, c_int, c_p, c_p, c_p, c_int, c_f, c_int, c_int, c_p]
        L.orc_maxpool.argtypes = [c_p, c_p, c_ll, c_int, c_int, c_p, c_p]
        L.orc_terminal_pool.argtypes = [c_p, c_p, c_int, c_int, c_int, c_p]
        L.orc_top_indices.argtypes = [c_p, c_int, c_int, c_p]
        L.orc_net_create.restype, L.orc_net_create.argtypes = c_p, [c_int] * 4
        L.orc_net_free.argtypes = [c_p]
        for n in ("orc_net_addLeNetLayerMP", "orc_net_addTriangularLeNetLayerMP"):
            getattr(L, n).argtypes = [c_p] + [c_int] * 6 + [c_f, c_int]
        L.orc_net_addLeNetLayerFMP.argtypes = [c_p] + [c_int] * 5 + [c_f, c_int, c_f, c_int]
        L.orc_net_set_fmp_seed.argtypes = [c_p, ctypes.c_uint]
        L.orc_net_set_dropout_features.restype, L.orc_net_set_dropout_features.argtypes = c_int, [c_p, c_int, c_p, c_int]
        L.orc_net_addTerminalPoolingLayer.argtypes = [c_p, c_int, c_int]
        L.orc_net_addSoftmaxLayer.argtypes = [c_p]
        L.orc_net_DeepCNet.restype = c_p
        L.orc_net_DeepCNet.argtypes = [c_int] * 6 + [c_f, c_int]
        L.orc_net_n_layers.restype, L.orc_net_n_layers.argtypes = c_int, [c_p]
        L.orc_net_input_spatial_size.restype, L.orc_net_input_spatial_size.argtypes = c_int, [c_p]
        L.orc_net_layer_info.argtypes = [c_p, c_int, c_p, c_p]
        L.orc_net_set_weights.argtypes = [c_p, c_int, c_p, c_p, c_p]
        L.orc_net_load_weights.restype, L.orc_net_load_weights.argtypes = c_int, [c_p, ctypes.c_char_p]
        L.orc_net_forward.argtypes = [c_p, c_int, c_p, c_p, c_p, c_int, c_int, c_int, c_p, c_p, c_p]
        L.orc_net_iface_sizes.argtypes = [c_p, c_int, c_p]
        L.orc_net_iface_fetch.argtypes = [c_p, c_int, c_p, c_p, c_p, c_p]
        L.orc_net_train_step.restype = c_int
        L.orc_net_train_step.argtypes = [c_p, c_int, c_p, c_p, c_p, c_p, c_f, c_f, c_int, c_p, c_p]
        L.orc_net_iface_dfeatures.restype, L.orc_net_iface_dfeatures.argtypes = c_ll, [c_p, c_int, c_p]
        L.orc_net_get_weights.argtypes = [c_p, c_int, c_p, c_p, c_p]
        L.orc_activation_backward.argtypes = [c_p, c_p, c_ll, c_int, c_int, c_p, c_p]
        L.orc_nin_backward.argtypes = [c_p, c_p, c_ll, c_int, c_int, c_p, c_p, c_p, c_p]
        L.orc_gather_backward.argtypes = [c_p, c_p, c_ll, c_int, c_ll, c_p]
        L.orc_maxpool_backward.argtypes = [c_p, c_p, c_ll, c_ll, c_p]
        L.orc_terminal_pool_backward.argtypes = [c_p, c_p, c_int, c_int, c_int, c_ll, c_p]
        L.orc_sgd_update.argtypes = [c_p, c_p, c_p, c_ll, c_f, c_f, c_int]

    # ---- fractional max-pooling
    def fmp_ticks(self, kind, dim, nIn, nOut, poolSize, seed, count):
        """Tick tables of `count` samples drawn from one RNG seeded with `seed`:
        [count, dim, 2*nOut + 2*nIn] = inputL, inputR, outputL, outputR per sample and axis."""
        out = np.zeros((count, dim, 2 * nOut + 2 * nIn), np.int32)
        f = self.lib.orc_fmp_ticks
        f.argtypes = [c_int] * 5 + [ctypes.c_uint, c_int, c_p]
        f(kind, dim, nIn, nOut, poolSize, seed, count, _p(out))
        return out

    def fmp_rules(self, dim, nIn, nOut, poolSize, overlapping, ticks, keys, rows, off, bg):
        keys, rows = np.ascontiguousarray(keys, np.int64), np.ascontiguousarray(rows, np.int32)
        off, bg = np.ascontiguousarray(off, np.int32), np.ascontiguousarray(bg, np.int32)
        ticks = np.ascontiguousarray(ticks, np.int32)
        f = self.lib.orc_fmp_rules
        f.restype, f.argtypes = c_p, [c_int] * 6 + [c_p] * 5
        h = f(dim, nIn, nOut, poolSize, int(overlapping), len(bg), _p(ticks), _p(keys), _p(rows), _p(off), _p(bg))
        return self._fetch(h, len(bg))

    # ---- layers
    def gather(self, feat, rules, nIn):
        feat = np.ascontiguousarray(feat, np.float32)
        rules = np.ascontiguousarray(rules, np.int32).ravel()
        out = np.zeros((rules.size, nIn), np.float32)
        self.lib.orc_gather(_p(feat), _p(rules), rules.size, nIn, _p(out))
        return out

    def nin_forward(self, X, W, B, prelu=None, p=1.0, act=NOSIGMOID, accum64=False):
        X = np.ascontiguousarray(X, np.float32)
        W = np.ascontiguousarray(W, np.float32)
        B = np.ascontiguousarray(B, np.float32)
        prelu = None if prelu is None else np.ascontiguousarray(prelu, np.float32)
        rows, K = X.shape
        N = W.shape[1]
        out = np.zeros((rows, N), np.float32)
        self.lib.orc_nin_forward(_p(X), rows, K, _p(W), _p(B), _p(prelu), N, p, act, int(accum64), _p(out))
        return out

    def maxpool(self, feat, rules, sd):
        feat = np.ascontiguousarray(feat, np.float32)
        rules = np.ascontiguousarray(rules, np.int32).reshape(-1, sd)
        C = feat.shape[1]
        out = np.zeros((rules.shape[0], C), np.float32)
        ch = np.zeros((rules.shape[0], C), np.int32)
        self.lib.orc_maxpool(_p(feat), _p(rules), rules.shape[0], sd, C, _p(out), _p(ch))
        return out, ch

    def terminal_pool(self, feat, rules, S):
        feat = np.ascontiguousarray(feat, np.float32)
        rules = np.ascontiguousarray(rules, np.int32).reshape(-1, S)
        C = feat.shape[1]
        out = np.zeros((rules.shape[0], C), np.float32)
        self.lib.orc_terminal_pool(_p(feat), _p(rules), rules.shape[0], S, C, _p(out))
        return out

    def top_indices(self, v, k):
        v = np.ascontiguousarray(v, np.float32)
        out = np.zeros(k, np.int32)
        self.lib.orc_top_indices(_p(v), len(v), k, _p(out))
        return out

    # ---- backward operations (fp64 accumulation)
    def activation_backward(self, out_features, d, act, prelu=None):
        """-> (d * f'(.) as a new array, slope gradient or None)."""
        b = np.ascontiguousarray(out_features, np.float32)
        d = np.array(d, np.float32, copy=True, order="C")
        rows, N = b.shape
        prelu = None if prelu is None else np.ascontiguousarray(prelu, np.float32)
        dpr = np.zeros(N, np.float32)
        self.lib.orc_activation_backward(_p(b), _p(d), rows, N, act, _p(prelu), _p(dpr))
        return d, (dpr if act == PRELU else None)

    def nin_backward(self, X, d, W, want_dx=True):
        """-> (dW [K x N], dB [N], dX [rows x K] or None)."""
        X, d, W = (np.ascontiguousarray(a, np.float32) for a in (X, d, W))
        rows, K = X.shape
        N = W.shape[1]
        dW, dB = np.zeros((K, N), np.float32), np.zeros(N, np.float32)
        dX = np.zeros((rows, K), np.float32) if want_dx else None
        self.lib.orc_nin_backward(_p(X), _p(d), rows, K, N, _p(W), _p(dW), _p(dB), _p(dX))
        return dW, dB, dX

    def gather_backward(self, d_conv, rules, nIn, rows_in):
        d_conv = np.ascontiguousarray(d_conv, np.float32)
        rules = np.ascontiguousarray(rules, np.int32).ravel()
        out = np.zeros((rows_in, nIn), np.float32)
        self.lib.orc_gather_backward(_p(d_conv), _p(rules), rules.size, nIn, rows_in, _p(out))
        return out

    def maxpool_backward(self, d_out, choices, n_in):
        d_out = np.ascontiguousarray(d_out, np.float32)
        choices = np.ascontiguousarray(choices, np.int32)
        out = np.zeros(n_in, np.float32)
        self.lib.orc_maxpool_backward(_p(d_out), _p(choices), d_out.size, n_in, _p(out))
        return out

    def terminal_pool_backward(self, d_out, rules, S, rows_in):
        d_out = np.ascontiguousarray(d_out, np.float32)
        rules = np.ascontiguousarray(rules, np.int32).reshape(-1, S)
        C = d_out.shape[1]
        out = np.zeros((rows_in, C), np.float32)
        self.lib.orc_terminal_pool_backward(_p(d_out), _p(rules), rules.shape[0], S, C, rows_in, _p(out))
        return out

    def sgd_update(self, w, m, d, lr, momentum, keep_positive=False):
        """NAG-light update in place on copies -> (w, m)."""
        w, m = np.array(w, np.float32, copy=True, order="C"), np.array(m, np.float32, copy=True, order="C")
        d = np.ascontiguousarray(d, np.float32)
        self.lib.orc_sgd_update(_p(w), _p(m), _p(d), w.size, lr, momentum, int(keep_positive))
        return w, m


class OracleNet:
    """Mirror of SparseConvNetCUDA's builder calls plus a CPU forward."""

    def __init__(self, oracle, dim, nInputFeatures, nClasses, nTop=1, handle=None, lattice=0):
        """lattice 0 mirrors SparseConvNet, 1 SparseConvTriangLeNet (SparseConvNet.h:20-99)."""
        self.o, self.L = oracle, oracle.lib
        self.dim, self.nIn, self.nClasses, self.nTop, self.lattice = dim, nInputFeatures, nClasses, nTop, lattice
        self.h = handle if handle is not None else self.L.orc_net_create(dim, nInputFeatures, nClasses, nTop)

    @classmethod
    def DeepCNet(cls, oracle, dim, l, k, fn, nInputFeatures, nClasses, p=0.0, nTop=1):
        h = oracle.lib.orc_net_DeepCNet(dim, l, k, fn, nInputFeatures, nClasses, p, nTop)
        return cls(oracle, dim, nInputFeatures, nClasses, nTop, handle=h)

    def __del__(self):
        try:
            self.L.orc_net_free(self.h)
        except Exception:
            pass

    def addLeNetLayerMP(self, nFeatures, fs, fstride, ps, pstride, act=RELU, dropout=0.0, minActive=1):
        f = self.L.orc_net_addTriangularLeNetLayerMP if self.lattice == 1 else self.L.orc_net_addLeNetLayerMP
        f(self.h, nFeatures, fs, fstride, ps, pstride, act, dropout, minActive)

    def addLeNetLayerFMP(self, kind, nFeatures, fs, fstride, ps, fmpShrink, act=RELU, dropout=0.0, minActive=1):
        self.L.orc_net_addLeNetLayerFMP(self.h, kind, nFeatures, fs, fstride, ps, fmpShrink, act, dropout, minActive)

    def seed_fmp(self, seed):
        """Every forward re-seeds FMP layer l's RNG with seed + l."""
        self.L.orc_net_set_fmp_seed(self.h, seed)

    def addTriangularLeNetLayerMP(self, nFeatures, fs, fstride, ps, pstride, act=RELU, dropout=0.0, minActive=1):
        self.L.orc_net_addTriangularLeNetLayerMP(self.h, nFeatures, fs, fstride, ps, pstride, act, dropout, minActive)

    def addTerminalPoolingLayer(self, poolSize, S=None):
        if S is None:  # the facades pass ipow / triangleSize (SparseConvNet.cu:56-58, 123-126)
            S = self.L.orc_triangleSize(poolSize, self.dim) if self.lattice == 1 else self.L.orc_ipow(poolSize, self.dim)
        self.L.orc_net_addTerminalPoolingLayer(self.h, poolSize, S)

    def addSoftmaxLayer(self):
        self.L.orc_net_addSoftmaxLayer(self.h)

    @property
    def inputSpatialSize(self):
        return self.L.orc_net_input_spatial_size(self.h)

    def layers(self):
        out = []
        for i in range(self.L.orc_net_n_layers(self.h)):
            info = np.zeros(10, np.int32)
            d = c_f()
            self.L.orc_net_layer_info(self.h, i, _p(info), ctypes.byref(d))
            keys = ("type", "size", "stride", "minActive", "nIn", "nOut", "fs", "act", "inSpatial", "outSpatial")
            rec = dict(zip(keys, (int(v) for v in info)))
            rec["dropout"] = float(d.value)
            out.append(rec)
        return out

    def set_weights(self, i, W, B, prelu=None):
        W = np.ascontiguousarray(W, np.float32)
        B = np.ascontiguousarray(B, np.float32)
        prelu = None if prelu is None else np.ascontiguousarray(prelu, np.float32)
        self.L.orc_net_set_weights(self.h, i, _p(W), _p(B), _p(prelu))

    def load_weights(self, path):
        rc = self.L.orc_net_load_weights(self.h, path.encode())
        if rc != 0:
            raise IOError("cannot read %s (%d)" % (path, rc))

    def forward(self, keys, off, features, threads=1, accum64=False, keep=False):
        """keys[row] (int64, -1 = background row), off[batch+1], features [rows x nIn].  keep retains every
        interface for iface(); with threads > 1 the batch is processed in that many sample chunks."""
        keys = np.ascontiguousarray(keys, np.int64)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        B = len(off) - 1
        probs = np.zeros((B, self.nClasses), np.float32)
        pred = np.zeros((B, self.nTop), np.int32)
        times = np.zeros(2, np.float64)
        self.L.orc_net_forward(self.h, B, _p(keys), _p(off), _p(features), threads, int(accum64), int(keep),
                               _p(probs), _p(pred), _p(times))
        self.times = times
        return probs, pred

    def set_dropout_features(self, layer, present):
        """The output features learnt layer `layer` keeps in the training steps that follow (ascending; empty: all)."""
        present = np.ascontiguousarray(present, np.int32)
        if self.L.orc_net_set_dropout_features(self.h, layer, _p(present), len(present)):
            raise ValueError("not a learnt layer, or more features than it has")

    def train_step(self, keys, off, features, labels, learning_rate, momentum, accum64=True):
        """One TRAINBATCH step (forward, SoftmaxClassifier, every layer's backwards with its SGD update) on a network
        without dropout -> (probabilities, dict(nll, mistakes)); interfaces and their dfeatures are kept."""
        keys = np.ascontiguousarray(keys, np.int64)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        labels = np.ascontiguousarray(labels, np.int32)
        B = len(off) - 1
        probs = np.zeros((B, self.nClasses), np.float32)
        stats = np.zeros(2, np.float64)
        rc = self.L.orc_net_train_step(self.h, B, _p(keys), _p(off), _p(features), _p(labels), learning_rate, momentum, int(accum64),
                                       _p(probs), _p(stats))
        if rc:
            raise ValueError("the oracle's training step needs a network without dropout")
        return probs, dict(nll=float(stats[0]), mistakes=int(stats[1]))

    def dfeatures(self, i):
        n = self.L.orc_net_iface_dfeatures(self.h, i, None)
        d = np.zeros(n, np.float32)
        self.L.orc_net_iface_dfeatures(self.h, i, _p(d))
        return d

    def get_weights(self, i):
        L = self.layers()[i]
        W, B = np.zeros((L["nIn"], L["nOut"]), np.float32), np.zeros(L["nOut"], np.float32)
        pr = np.zeros(L["nOut"], np.float32)
        self.L.orc_net_get_weights(self.h, i, _p(W), _p(B), _p(pr))
        return W, B, (pr if L["act"] == PRELU else None)

    def iface(self, i):
        """Interface i of the last forward(keep=True): 0 is the input, i+1 layer i's output."""
        s = np.zeros(5, np.int64)
        self.L.orc_net_iface_sizes(self.h, i, _p(s))
        rows, nF, sp, nr, nc = (int(v) for v in s)
        feat = np.zeros((rows, nF), np.float32)
        rules = np.zeros(nr, np.int32)
        ch = np.zeros(nc, np.int32)
        rk = np.zeros(rows, np.int64)
        self.L.orc_net_iface_fetch(self.h, i, _p(feat), _p(rules), _p(ch), _p(rk))
        return dict(nSpatialSites=rows, nFeatures=nF, spatialSize=sp, features=feat, rules=rules,
                    choices=ch, row_keys=rk)
