"""ai.onnx.ml operators against scikit-learn models / numpy restatements, plus TfIdfVectorizer, STFT, MelWeightMatrix,
MaxRoiPool, Optional* and GatherBlockQuantized against restatements of their specifications."""
import numpy as np
import pytest
import torch

from helpers import run_node

ML = "ai.onnx.ml"
MS = "com.microsoft"
rng = np.random.default_rng(0)


def _tree_attrs(trees, prefix, leaf_weights):
    """scikit-learn trees -> the nodes_* / <prefix>_* attributes.  leaf_weights(tree, node) -> [(output id, weight)]."""
    a = {k: [] for k in ("nodes_treeids", "nodes_nodeids", "nodes_featureids", "nodes_values", "nodes_modes", "nodes_truenodeids",
                         "nodes_falsenodeids", f"{prefix}_treeids", f"{prefix}_nodeids", f"{prefix}_ids", f"{prefix}_weights")}
    for t, tree in enumerate(trees):
        tr = tree.tree_
        for i in range(tr.node_count):
            leaf = tr.children_left[i] < 0
            a["nodes_treeids"].append(t)
            a["nodes_nodeids"].append(i)
            a["nodes_featureids"].append(0 if leaf else int(tr.feature[i]))
            a["nodes_values"].append(0.0 if leaf else float(tr.threshold[i]))
            a["nodes_modes"].append("LEAF" if leaf else "BRANCH_LEQ")
            a["nodes_truenodeids"].append(0 if leaf else int(tr.children_left[i]))
            a["nodes_falsenodeids"].append(0 if leaf else int(tr.children_right[i]))
            if leaf:
                for out_id, w in leaf_weights(tr, i):
                    a[f"{prefix}_treeids"].append(t)
                    a[f"{prefix}_nodeids"].append(i)
                    a[f"{prefix}_ids"].append(int(out_id))
                    a[f"{prefix}_weights"].append(float(w))
    return a


def _data(n=200, f=6):
    X = rng.integers(0, 20, (n, f)).astype(np.float32)    # integer grid: split thresholds k + 0.5 are exact in float32
    return X


def test_tree_ensemble_regressor_matches_random_forest():
    from sklearn.ensemble import RandomForestRegressor
    X = _data()
    y = np.stack([X[:, 0] * 2 - X[:, 1] + np.sin(X[:, 2]), X[:, 3] - X[:, 4]], 1)
    m = RandomForestRegressor(n_estimators=7, max_depth=5, random_state=0).fit(X, y)
    attrs = _tree_attrs(m.estimators_, "target", lambda tr, i: [(k, tr.value[i, k, 0]) for k in range(2)])
    (out,) = run_node("TreeEnsembleRegressor", {"X": X}, domain=ML, n_targets=2, aggregate_function="AVERAGE", **attrs)
    np.testing.assert_allclose(out, m.predict(X), rtol=1e-5, atol=1e-5)
    # SUM with base values
    (out,) = run_node("TreeEnsembleRegressor", {"X": X}, domain=ML, n_targets=2, base_values=[1.0, -2.0], **attrs)
    np.testing.assert_allclose(out, m.predict(X) * 7 + np.array([1.0, -2.0]), rtol=1e-5, atol=1e-4)


def test_tree_ensemble_regressor_min_max_and_modes():
    # two hand-made stumps using different comparison modes; missing values follow the tracked branch
    attrs = dict(nodes_treeids=[0, 0, 0, 1, 1, 1], nodes_nodeids=[0, 1, 2, 0, 1, 2], nodes_featureids=[0, 0, 0, 1, 0, 0],
                 nodes_values=[2.0, 0.0, 0.0, 5.0, 0.0, 0.0], nodes_modes=["BRANCH_GT", "LEAF", "LEAF", "BRANCH_EQ", "LEAF", "LEAF"],
                 nodes_truenodeids=[1, 0, 0, 1, 0, 0], nodes_falsenodeids=[2, 0, 0, 2, 0, 0], nodes_missing_value_tracks_true=[1, 0, 0, 0, 0, 0],
                 target_treeids=[0, 0, 1, 1], target_nodeids=[1, 2, 1, 2], target_ids=[0, 0, 0, 0], target_weights=[10.0, -1.0, 3.0, 4.0])
    X = np.array([[3, 5], [1, 5], [3, 4], [np.nan, 4]], np.float32)
    t0 = np.array([10, -1, 10, 10.0])
    t1 = np.array([3, 3, 4, 4.0])
    for agg, ref in (("SUM", t0 + t1), ("MIN", np.minimum(t0, t1)), ("MAX", np.maximum(t0, t1)), ("AVERAGE", (t0 + t1) / 2)):
        (out,) = run_node("TreeEnsembleRegressor", {"X": X}, domain=ML, n_targets=1, aggregate_function=agg, **attrs)
        np.testing.assert_allclose(out[:, 0], ref, rtol=1e-6)


def test_tree_ensemble_classifier_matches_random_forest():
    from sklearn.ensemble import RandomForestClassifier
    X = _data()
    y = (X[:, 0] + X[:, 1] > 20).astype(np.int64) + (X[:, 2] > 10)
    m = RandomForestClassifier(n_estimators=5, max_depth=4, random_state=1).fit(X, y)
    def weights(tr, i):
        v = tr.value[i, 0]
        v = v / v.sum()
        return [(k, v[k] / 5) for k in range(3)]
    attrs = _tree_attrs(m.estimators_, "class", weights)
    labels, scores = run_node("TreeEnsembleClassifier", {"X": X}, n_outputs=2, domain=ML, classlabels_int64s=[10, 11, 12], **attrs)
    proba = m.predict_proba(X)
    np.testing.assert_allclose(scores, proba, rtol=1e-5, atol=1e-6)
    clear = np.sort(proba, 1)[:, -1] - np.sort(proba, 1)[:, -2] > 1e-6
    np.testing.assert_array_equal(labels[clear], m.predict(X)[clear] + 10)


def test_tree_ensemble_classifier_binary_single_score_logistic():
    from sklearn.ensemble import GradientBoostingClassifier
    X = _data()
    y = (X[:, 0] - X[:, 3] + rng.normal(0, 2, len(X)) > 0).astype(np.int64)
    m = GradientBoostingClassifier(n_estimators=8, max_depth=3, learning_rate=0.3, random_state=0).fit(X, y)
    trees = [e[0] for e in m.estimators_]
    attrs = _tree_attrs(trees, "class", lambda tr, i: [(0, 0.3 * tr.value[i, 0, 0])])
    prior = m.init_.class_prior_[1]
    base = float(np.log(prior / (1 - prior)))
    labels, scores = run_node("TreeEnsembleClassifier", {"X": X}, n_outputs=2, domain=ML, classlabels_int64s=[0, 1], base_values=[base],
                              post_transform="LOGISTIC", **attrs)
    np.testing.assert_allclose(scores, m.predict_proba(X), rtol=1e-4, atol=1e-6)
    np.testing.assert_array_equal(labels, m.predict(X))


def test_linear_regressor_and_classifier():
    X = rng.standard_normal((9, 4)).astype(np.float32)
    W = rng.standard_normal((3, 4)).astype(np.float32)
    b = rng.standard_normal(3).astype(np.float32)
    s = X @ W.T + b
    (y,) = run_node("LinearRegressor", {"X": X}, domain=ML, coefficients=W.ravel().tolist(), intercepts=b.tolist(), targets=3)
    np.testing.assert_allclose(y, s, rtol=1e-5, atol=1e-5)
    labels, scores = run_node("LinearClassifier", {"X": X}, n_outputs=2, domain=ML, coefficients=W.ravel().tolist(), intercepts=b.tolist(),
                              classlabels_ints=[5, 6, 7], post_transform="SOFTMAX")
    e = np.exp(s - s.max(1, keepdims=True))
    np.testing.assert_allclose(scores, e / e.sum(1, keepdims=True), rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(labels, s.argmax(1) + 5)
    # a single row of coefficients with two labels is a binary model
    labels, scores = run_node("LinearClassifier", {"X": X}, n_outputs=2, domain=ML, coefficients=W[0].tolist(), intercepts=[float(b[0])],
                              classlabels_ints=[0, 1], post_transform="LOGISTIC")
    p = 1 / (1 + np.exp(-s[:, 0]))
    np.testing.assert_allclose(scores, np.stack([1 - p, p], 1), rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(labels, (s[:, 0] > 0).astype(np.int64))


@pytest.mark.parametrize("kernel", ["linear", "rbf", "poly", "sigmoid"])
def test_svm_regressor_matches_sklearn(kernel):
    from sklearn.svm import SVR
    X = rng.standard_normal((60, 3)).astype(np.float32)
    y = X[:, 0] * 2 + np.tanh(X[:, 1]) - X[:, 2] ** 2
    m = SVR(kernel=kernel, gamma=0.4, coef0=0.3, degree=3, C=2.0).fit(X.astype(np.float64), y)
    (out,) = run_node("SVMRegressor", {"X": X}, domain=ML, kernel_type=kernel.upper(), kernel_params=[0.4, 0.3, 3.0],
                      n_supports=len(m.support_vectors_), support_vectors=m.support_vectors_.ravel().tolist(),
                      coefficients=m.dual_coef_.ravel().tolist(), rho=[float(m.intercept_[0])])
    np.testing.assert_allclose(out[:, 0], m.predict(X.astype(np.float64)), rtol=1e-3, atol=1e-3)


def test_feature_transforms():
    X = rng.standard_normal((5, 4)).astype(np.float32)
    (y,) = run_node("Scaler", {"X": X}, domain=ML, offset=[1.0, 2.0, 3.0, 4.0], scale=[0.5, 2.0, 1.0, -1.0])
    np.testing.assert_allclose(y, (X - [1, 2, 3, 4]) * [0.5, 2, 1, -1], rtol=1e-6)
    for norm, d in (("MAX", np.abs(X).max(1)), ("L1", np.abs(X).sum(1)), ("L2", np.sqrt((X ** 2).sum(1)))):
        (y,) = run_node("Normalizer", {"X": X}, domain=ML, norm=norm)
        np.testing.assert_allclose(y, X / d[:, None], rtol=1e-5)
    (y,) = run_node("Binarizer", {"X": X}, domain=ML, threshold=0.25)
    np.testing.assert_array_equal(y, (X > 0.25).astype(np.float32))
    Xn = X.copy()
    Xn[0, 1] = Xn[3, 2] = np.nan
    (y,) = run_node("Imputer", {"X": Xn}, domain=ML, imputed_value_floats=[9.0, 8.0, 7.0, 6.0], replaced_value_float=float("nan"))
    ref = Xn.copy()
    ref[0, 1], ref[3, 2] = 8.0, 7.0
    np.testing.assert_array_equal(y, ref)
    xi = np.array([[1, -1], [-1, 5]], np.int64)
    (y,) = run_node("Imputer", {"X": xi}, domain=ML, imputed_value_int64s=[42], replaced_value_int64=-1)
    np.testing.assert_array_equal(y, [[1, 42], [42, 5]])
    cats = np.array([[3, 9], [4, 7]], np.int64)
    (y,) = run_node("OneHotEncoder", {"X": cats}, domain=ML, cats_int64s=[3, 4, 9], zeros=1)
    np.testing.assert_array_equal(y, [[[1, 0, 0], [0, 0, 1]], [[0, 1, 0], [0, 0, 0]]])
    (y,) = run_node("ArrayFeatureExtractor", {"X": X, "Y": np.array([3, 0], np.int64)}, domain=ML)
    np.testing.assert_array_equal(y, X[:, [3, 0]])
    a, b = X[:, :2], np.arange(15, dtype=np.int64).reshape(5, 3)
    (y,) = run_node("FeatureVectorizer", {"a": a, "b": b}, domain=ML, inputdimensions=[2, 3])
    np.testing.assert_allclose(y, np.concatenate([a, b.astype(np.float32)], 1))


def test_tfidf_vectorizer_spec_examples():
    # the ONNX specification's worked examples (uni- and bi-grams with skips)
    x = np.array([[1, 1, 3, 3, 3, 7], [8, 6, 7, 5, 6, 8]], np.int32)
    common = dict(ngram_counts=[0, 4], ngram_indexes=[0, 1, 2, 3, 4, 5, 6], pool_int64s=[2, 3, 5, 4, 5, 6, 7, 8, 6, 7])
    (y,) = run_node("TfIdfVectorizer", {"X": x}, mode="TF", min_gram_length=2, max_gram_length=2, max_skip_count=0, **common)
    np.testing.assert_array_equal(y, [[0, 0, 0, 0, 0, 0, 0], [0, 0, 0, 0, 1, 0, 1]])
    (y,) = run_node("TfIdfVectorizer", {"X": x}, mode="TF", min_gram_length=1, max_gram_length=2, max_skip_count=5, **common)
    np.testing.assert_array_equal(y, [[0, 3, 0, 0, 0, 0, 0], [0, 0, 1, 0, 1, 1, 1]])
    (y,) = run_node("TfIdfVectorizer", {"X": x.ravel()[:12]}, mode="IDF", min_gram_length=1, max_gram_length=2, max_skip_count=5,
                    weights=[1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0], **common)
    flat = x.ravel()
    tf = np.zeros(7)
    pool1, pool2 = [2, 3, 5, 4], [(5, 6), (7, 8), (6, 7)]
    for i, v in enumerate(pool1):
        tf[i] = (flat == v).sum()
    for j, (p, q) in enumerate(pool2):
        tf[4 + j] = sum(1 for s in range(6) for i in range(12 - s - 1) if flat[i] == p and flat[i + s + 1] == q)
    np.testing.assert_array_equal(y, np.where(tf > 0, np.arange(1, 8), 0))


def test_stft_and_mel_weight_matrix():
    sig = rng.standard_normal((2, 64, 1)).astype(np.float32)
    win = np.hanning(16).astype(np.float32)
    (y,) = run_node("STFT", {"signal": sig, "step": np.array(8, np.int64), "window": win, "len": np.array(16, np.int64)})
    frames = np.stack([sig[:, s:s + 16, 0] * win for s in range(0, 64 - 16 + 1, 8)], 1)
    ref = np.fft.rfft(frames, axis=-1)
    np.testing.assert_allclose(y, np.stack([ref.real, ref.imag], -1), rtol=1e-4, atol=1e-4)
    (y2,) = run_node("STFT", {"signal": sig, "step": np.array(8, np.int64), "window": None, "len": np.array(16, np.int64)}, onesided=0)
    ref2 = np.fft.fft(np.stack([sig[:, s:s + 16, 0] for s in range(0, 49, 8)], 1), axis=-1)
    np.testing.assert_allclose(y2, np.stack([ref2.real, ref2.imag], -1), rtol=1e-4, atol=1e-4)

    mels, dft, rate, lo, hi = 8, 16, 8192, 0.0, 4096.0
    (m,) = run_node("MelWeightMatrix", {"m": np.array(mels, np.int64), "d": np.array(dft, np.int64), "r": np.array(rate, np.int64),
                                         "lo": np.array(lo, np.float32), "hi": np.array(hi, np.float32)})
    # expected matrix of the reference's own test (onnxruntime/test/providers/cpu/signal/signal_ops_test.cc, MelWeightMatrixFloat)
    ref = np.zeros((9, 8), np.float32)
    for row, col in ((0, 0), (0, 1), (1, 2), (1, 3), (2, 4), (3, 5), (4, 6), (5, 7)):
        ref[row, col] = 1
    np.testing.assert_array_equal(m, ref)


def test_max_roi_pool():
    x = rng.standard_normal((2, 3, 8, 8)).astype(np.float32)
    rois = np.array([[0, 0, 0, 7, 7], [1, 2, 2, 5, 5], [0, 1, 3, 2, 6]], np.float32)
    (y,) = run_node("MaxRoiPool", {"X": x, "rois": rois}, pooled_shape=[2, 2], spatial_scale=1.0)
    assert y.shape == (3, 3, 2, 2)
    np.testing.assert_allclose(y[0], torch.nn.functional.max_pool2d(torch.from_numpy(x[0]), 4).numpy())
    np.testing.assert_allclose(y[1], torch.nn.functional.max_pool2d(torch.from_numpy(x[1, :, 2:6, 2:6]), 2).numpy())
    np.testing.assert_allclose(y[2, :, 0, 0], x[0, :, 3:5, 1:2].max((1, 2)))
    np.testing.assert_allclose(y[2, :, 1, 1], x[0, :, 5:7, 2:3].max((1, 2)))


def test_optional_ops():
    x = rng.standard_normal((2, 3)).astype(np.float32)
    (y,) = run_node("Optional", {"x": x}, opset=18)
    np.testing.assert_array_equal(y, x)
    (y,) = run_node("OptionalGetElement", {"x": x}, opset=18)
    np.testing.assert_array_equal(y, x)
    (h,) = run_node("OptionalHasElement", {"x": x}, opset=18)
    assert bool(h) is True
    (h,) = run_node("OptionalHasElement", {"x": None}, opset=18)
    assert bool(h) is False


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_gather_block_quantized(bits):
    rows, K, block = 10, 64, 16
    per = 8 // bits
    q = rng.integers(0, 1 << bits, (rows, K)).astype(np.uint8)
    zp = rng.integers(0, 1 << bits, (rows, K // block)).astype(np.uint8)
    def pack(v):
        pad = (-v.shape[1]) % per
        v = np.pad(v, ((0, 0), (0, pad))).reshape(v.shape[0], -1, per).astype(np.uint32)
        return sum(v[:, :, k] << (k * bits) for k in range(per)).astype(np.uint8)
    scales = (rng.random((rows, K // block)) + 0.5).astype(np.float32)
    idx = np.array([[3, 0], [9, -1]], np.int64)
    (y,) = run_node("GatherBlockQuantized", {"data": pack(q), "indices": idx, "scales": scales, "zp": pack(zp)}, domain=MS,
                    bits=bits, block_size=block, gather_axis=0, quantize_axis=1)
    deq = (q.astype(np.float32) - np.repeat(zp, block, 1)) * np.repeat(scales, block, 1)
    np.testing.assert_allclose(y, deq[idx], rtol=1e-6)
    (y,) = run_node("GatherBlockQuantized", {"data": pack(q), "indices": idx, "scales": scales, "zp": None}, domain=MS,
                    bits=bits, block_size=block)
    deq = (q.astype(np.float32) - (1 << (bits - 1))) * np.repeat(scales, block, 1)
    np.testing.assert_allclose(y, deq[idx], rtol=1e-6)


def _svc_attrs(m, negate):
    sign = -1.0 if negate else 1.0     # scikit-learn flips the sign of a two-class model; the operator wants libsvm's
    return dict(kernel_type=m.kernel.upper(), kernel_params=[float(m._gamma), float(m.coef0), float(m.degree)],
                support_vectors=m.support_vectors_.ravel().tolist(), vectors_per_class=[int(v) for v in m.n_support_],
                coefficients=(sign * m.dual_coef_).ravel().tolist(), rho=(sign * m.intercept_).tolist())


@pytest.mark.parametrize("kernel", ["rbf", "linear", "poly"])
def test_svm_classifier_multiclass_matches_sklearn(kernel):
    from sklearn.svm import SVC
    X = rng.standard_normal((150, 4))
    y = (X[:, 0] > 0.3).astype(int) + (X[:, 1] + X[:, 2] > 0.5).astype(int) * 2
    m = SVC(kernel=kernel, gamma=0.3, coef0=0.5, degree=2, decision_function_shape="ovo").fit(X, y)
    labels, scores = run_node("SVMClassifier", {"X": X.astype(np.float32)}, n_outputs=2, domain=ML,
                              classlabels_ints=[int(c) for c in m.classes_], **_svc_attrs(m, False))
    dec = m.decision_function(X.astype(np.float32).astype(np.float64))
    np.testing.assert_allclose(scores, dec, rtol=2e-3, atol=2e-3)
    clear = np.abs(dec).min(1) > 1e-3
    np.testing.assert_array_equal(labels[clear], m.predict(X.astype(np.float32).astype(np.float64))[clear])


def test_svm_classifier_binary_probabilities_and_string_labels():
    from sklearn.svm import SVC
    X = rng.standard_normal((120, 3))
    y2 = (X[:, 0] + 0.5 * X[:, 1] > 0).astype(int)
    m = SVC(kernel="rbf", gamma=0.5).fit(X, y2)
    Xf = X.astype(np.float32)
    labels, scores = run_node("SVMClassifier", {"X": Xf}, n_outputs=2, domain=ML, classlabels_strings=["neg", "pos"], **_svc_attrs(m, True))
    dec = m.decision_function(Xf.astype(np.float64))
    np.testing.assert_allclose(scores, np.stack([dec, -dec], 1), rtol=2e-3, atol=2e-3)      # [-d, d] with d = libsvm's decision
    clear = np.abs(dec) > 1e-3
    assert labels.dtype == object
    np.testing.assert_array_equal(labels[clear], np.where(m.predict(Xf.astype(np.float64)) == 1, "pos", "neg")[clear])
    # three classes with Platt scaling: pairwise probabilities coupled into class probabilities
    y3 = (X[:, 0] > 0.3).astype(int) + (X[:, 1] > 0.2).astype(int)
    mp = SVC(kernel="rbf", gamma=0.5, probability=True, random_state=0).fit(X, y3)
    labels, scores = run_node("SVMClassifier", {"X": Xf}, n_outputs=2, domain=ML, classlabels_ints=[0, 1, 2],
                              prob_a=mp.probA_.tolist(), prob_b=mp.probB_.tolist(), **_svc_attrs(mp, False))
    np.testing.assert_allclose(scores, mp.predict_proba(Xf.astype(np.float64)), rtol=5e-3, atol=5e-3)


def test_linear_and_tree_classifiers_with_string_labels():
    X = rng.standard_normal((6, 3)).astype(np.float32)
    W = rng.standard_normal((3, 3)).astype(np.float32)
    labels, _ = run_node("LinearClassifier", {"X": X}, n_outputs=2, domain=ML, coefficients=W.ravel().tolist(), intercepts=[0.0, 0.0, 0.0],
                         classlabels_strings=["a", "b", "c"])
    assert labels.tolist() == [["a", "b", "c"][i] for i in (X @ W.T).argmax(1)]
    attrs = dict(nodes_treeids=[0, 0, 0], nodes_nodeids=[0, 1, 2], nodes_featureids=[0, 0, 0], nodes_values=[0.0, 0.0, 0.0],
                 nodes_modes=["BRANCH_LEQ", "LEAF", "LEAF"], nodes_truenodeids=[1, 0, 0], nodes_falsenodeids=[2, 0, 0],
                 class_treeids=[0, 0], class_nodeids=[1, 2], class_ids=[0, 1], class_weights=[1.0, 1.0])
    labels, scores = run_node("TreeEnsembleClassifier", {"X": X}, n_outputs=2, domain=ML, classlabels_strings=["low", "high"], **attrs)
    assert labels.tolist() == ["low" if v <= 0 else "high" for v in X[:, 0]]


def test_zipmap_returns_a_list_of_dicts():
    X = np.array([[0.1, 0.9], [0.75, 0.25]], np.float32)
    (rows,) = run_node("ZipMap", {"X": X}, domain=ML, classlabels_int64s=[10, 20])
    assert isinstance(rows, list) and len(rows) == 2 and set(rows[0]) == {10, 20}
    assert rows[1][10] == pytest.approx(0.75) and rows[0][20] == pytest.approx(0.9)
    (rows,) = run_node("ZipMap", {"X": X[0]}, domain=ML, classlabels_strings=["no", "yes"])
    assert rows == [{"no": pytest.approx(0.1), "yes": pytest.approx(0.9)}]
    # the usual tail of a converted scikit-learn classifier: classifier -> ZipMap on the probabilities
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    from helpers import graph_model
    W = np.array([[1.0, -1.0], [-1.0, 1.0]], np.float32)
    nodes = [ol.make_node("LinearClassifier", ["X"], ["label", "proba"], domain=ML, coefficients=W.ravel().tolist(), intercepts=[0.0, 0.0],
                          classlabels_strings=["a", "b"], post_transform="SOFTMAX"),
             ol.make_node("ZipMap", ["proba"], ["probs"], domain=ML, classlabels_strings=["a", "b"])]
    model = graph_model(nodes, [ol.make_tensor_value_info("X", ol.TensorProto.FLOAT, ["n", 2])],
                        [ol.make_tensor_value_info("label", ol.TensorProto.STRING, None), ol.make_tensor_value_info("probs", 0, None)])
    label, probs = ort.InferenceSession(model, providers=["CPUExecutionProvider"]).run(None, {"X": np.array([[2.0, 0.0], [0.0, 3.0]], np.float32)})
    assert label.tolist() == ["a", "b"] and probs[0]["a"] > 0.9 and probs[1]["b"] > 0.9


def test_tree_ensemble_opset5_spec_examples():
    """ai.onnx.ml TreeEnsemble (opset 5): one tree with set-membership nodes, and one with plain <= splits (the attribute
    sets of the specification's examples; expected values worked out by hand)."""
    from onnxruntime_b200 import onnx_lite as ol
    import onnxruntime_b200 as ort
    def run(x, **attrs):
        node = ol.make_node("TreeEnsemble", ["X"], ["Y"], domain=ML, **attrs)
        g = ol.make_graph([node], "g", [ol.make_tensor_value_info("X", ol.TensorProto.FLOAT, list(x.shape))], [ol.make_tensor_value_info("Y", 0, None)])
        m = ol.make_model(g, opset=17)
        m.opset_imports[ML] = 5
        return ort.InferenceSession(m.serialize(), providers=["CPUExecutionProvider"]).run(None, {"X": x})[0]
    x = np.array([1.2, 3.4, -0.12, 12, 7, 9], np.float32).reshape(-1, 1)
    y = run(x, n_targets=2, aggregate_function=1, membership_values=np.array([1.2, 3.7, 8, 9, np.nan, 12, 7, np.nan], np.float32),
            nodes_missing_value_tracks_true=[0, 0, 0], nodes_hitrates=np.array([1, 1, 1], np.float32), post_transform=0, tree_roots=[0],
            nodes_modes=np.array([0, 6, 6], np.uint8), nodes_featureids=[0, 0, 0], nodes_splits=np.array([11, 232344.0, np.nan], np.float32),
            nodes_trueleafs=[0, 1, 1], nodes_truenodeids=[1, 0, 1], nodes_falseleafs=[1, 0, 1], nodes_falsenodeids=[2, 2, 3],
            leaf_targetids=[0, 1, 0, 1], leaf_weights=np.array([1, 10, 1000, 100], np.float32))
    # node 0: x <= 11 ? node 1 : leaf 2;  node 1: x in {1.2, 3.7, 8, 9} ? leaf 0 : node 2;  node 2: x in {12, 7} ? leaf 1 : leaf 3
    np.testing.assert_array_equal(y, [[1, 0], [0, 100], [0, 100], [1000, 0], [0, 10], [1, 0]])
    x = np.array([[1.2, 3.4, -0.12], [-0.67, 0.88, 1.29], [4.5, 0.9, 2.11]], np.float32)
    y = run(x, n_targets=2, aggregate_function=1, nodes_missing_value_tracks_true=[0, 0, 0], post_transform=0, tree_roots=[0],
            nodes_modes=np.array([0, 0, 0], np.uint8), nodes_featureids=[0, 0, 0], nodes_splits=np.array([3.14, 1.2, 4.2], np.float32),
            nodes_trueleafs=[0, 1, 1], nodes_truenodeids=[1, 0, 1], nodes_falseleafs=[0, 1, 1], nodes_falsenodeids=[2, 2, 3],
            leaf_targetids=[0, 1, 0, 1], leaf_weights=np.array([5.23, 12.12, -12.23, 7.21], np.float32))
    # node 0: x0 <= 3.14 ? node 1 : node 2;  node 1: x0 <= 1.2 ? leaf 0 : leaf 2;  node 2: x0 <= 4.2 ? leaf 1 : leaf 3
    np.testing.assert_allclose(y, [[5.23, 0], [5.23, 0], [0, 7.21]], rtol=1e-6)


def test_cast_map_and_dict_vectorizer_take_python_dicts():
    (y,) = run_node("DictVectorizer", {"X": {"b": 2.5, "zz": 9.0, "a": 1.0}}, domain=ML, string_vocabulary=["a", "b", "c"])
    np.testing.assert_array_equal(y, [[1.0, 2.5, 0.0]])
    (y,) = run_node("DictVectorizer", {"X": {7: 0.5, 3: 4.0}}, domain=ML, int64_vocabulary=[3, 5, 7])
    np.testing.assert_array_equal(y, [[4.0, 0.0, 0.5]])
    (y,) = run_node("CastMap", {"X": {4: "2.5", 1: "7"}}, domain=ML, cast_to="TO_FLOAT", map_form="DENSE")
    np.testing.assert_array_equal(y, [[7.0, 2.5]])
    (y,) = run_node("CastMap", {"X": {4: 2.0, 1: 7.0}}, domain=ML, cast_to="TO_INT64", map_form="SPARSE", max_map=6)
    np.testing.assert_array_equal(y, [[0, 7, 0, 0, 2, 0]])
    (y,) = run_node("CastMap", {"X": {0: 1.5, 2: 3.0}}, domain=ML, cast_to="TO_STRING", map_form="DENSE")
    assert y.tolist() == [["1.5", "3"]]
