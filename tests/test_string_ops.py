"""Tensors of strings: feeds, outputs, initializers and Constant nodes; the string operators; operators that only move
elements applied to strings; numeric <-> string casts; string forms of LabelEncoder / CategoryMapper / OneHotEncoder /
TfIdfVectorizer; the contrib Tokenizer.  Expected values are the worked examples of the ONNX operator specifications."""
import numpy as np
import pytest

import onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol
from helpers import run_node, graph_model

T = ol.TensorProto
ML = "ai.onnx.ml"
MS = "com.microsoft"


def S(*items, shape=None):
    a = np.empty(len(items), dtype=object)
    a[:] = items
    return a.reshape(shape) if shape is not None else a


def test_string_feed_identity_and_metadata():
    model = graph_model([ol.make_node("Identity", ["x"], ["y"])], [ol.make_tensor_value_info("x", T.STRING, ["n", 2])],
                        [ol.make_tensor_value_info("y", T.STRING, None)])
    sess = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    assert sess.get_inputs()[0].type == "tensor(string)"
    x = S("a", "bc", "", "déjà vu", shape=(2, 2))
    (y,) = sess.run(None, {"x": x})
    assert y.dtype == object and y.shape == (2, 2) and y.tolist() == x.tolist()
    (y,) = sess.run(None, {"x": np.array([["p", "q"]])})          # numpy unicode arrays are accepted too
    assert y.tolist() == [["p", "q"]]
    with pytest.raises(Exception, match="Unexpected input data type"):
        sess.run(None, {"x": np.zeros((1, 2), np.int64)})


def test_string_initializer_constant_gather_concat_and_saved_model(tmp_path):
    vocab = ol.make_tensor("vocab", S("zero", "one", "two", "three"))
    nodes = [ol.make_node("Gather", ["vocab", "idx"], ["words"]),
             ol.make_node("Constant", [], ["tail"], value_strings=["<end>"]),
             ol.make_node("Concat", ["words", "tail"], ["y"], axis=0)]
    model = graph_model(nodes, [ol.make_tensor_value_info("idx", T.INT64, ["n"])], [ol.make_tensor_value_info("y", T.STRING, None)], [vocab])
    so = ort.SessionOptions()
    so.optimized_model_filepath = str(tmp_path / "opt.onnx")
    sess = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    (y,) = sess.run(None, {"idx": np.array([3, 0, 2], np.int64)})
    assert y.tolist() == ["three", "zero", "two", "<end>"]
    again = ort.InferenceSession(str(tmp_path / "opt.onnx"), providers=["CPUExecutionProvider"])      # strings survive serialisation
    assert again.run(None, {"idx": np.array([1], np.int64)})[0].tolist() == ["one", "<end>"]


def test_string_normalizer():
    x = S("monday", "tuesday", "wednesday", "thursday")
    (y,) = run_node("StringNormalizer", {"x": x}, case_change_action="UPPER", stopwords=["monday"])
    assert y.tolist() == ["TUESDAY", "WEDNESDAY", "THURSDAY"]
    (y,) = run_node("StringNormalizer", {"x": S("Monday", "tuesday", "MONDAY")}, case_change_action="LOWER", stopwords=["monday"], is_case_sensitive=0)
    assert y.tolist() == ["tuesday"]
    (y,) = run_node("StringNormalizer", {"x": S("Monday", "monday")}, stopwords=["monday"], is_case_sensitive=1)
    assert y.tolist() == ["Monday"]
    (y,) = run_node("StringNormalizer", {"x": S("monday", "monday", shape=(1, 2))}, stopwords=["monday"])
    assert y.shape == (1, 1) and y.tolist() == [[""]]


def test_string_concat_split_regex():
    (y,) = run_node("StringConcat", {"a": S("abc", "def"), "b": S(".com", ".net")}, opset=20)
    assert y.tolist() == ["abc.com", "def.net"]
    (y,) = run_node("StringConcat", {"a": S("x", "y", shape=(2, 1)), "b": S("1", "2", "3")}, opset=20)
    assert y.tolist() == [["x1", "x2", "x3"], ["y1", "y2", "y3"]]
    y, z = run_node("StringSplit", {"x": S("hello world", "def  ghi jkl", "")}, n_outputs=2, opset=20)
    assert y.tolist() == [["hello", "world", ""], ["def", "ghi", "jkl"], ["", "", ""]] and z.tolist() == [2, 3, 0]
    y, z = run_node("StringSplit", {"x": S("a,b,,c", "x")}, n_outputs=2, opset=20, delimiter=",", maxsplit=2)
    assert y.tolist() == [["a", "b", ",c"], ["x", "", ""]] and z.tolist() == [3, 1]
    (m,) = run_node("RegexFullMatch", {"x": S("www.google.com", "www.facebook.com", "www.bbc.co.uk")}, opset=20, pattern=r"www\.[\w.-]+\.\bcom\b")
    assert m.dtype == np.bool_ and m.tolist() == [True, True, False]


def test_cast_between_strings_and_numbers():
    (y,) = run_node("Cast", {"x": S("0.47", "-3", "1e3", "INF", shape=(2, 2))}, to=T.FLOAT)
    np.testing.assert_array_equal(y, np.array([[0.47, -3.0], [1000.0, np.inf]], np.float32))
    (y,) = run_node("Cast", {"x": np.array([0.5, 3.0, 1e-7, np.nan], np.float32)}, to=T.STRING)
    assert y.tolist() == ["0.5", "3", "1e-07", "NaN"]
    (y,) = run_node("Cast", {"x": np.array([12, -7], np.int64)}, to=T.STRING)
    assert y.tolist() == ["12", "-7"]
    (y,) = run_node("Cast", {"x": S("42")}, to=T.INT64)
    assert y.dtype == np.int64 and y.tolist() == [42]


def test_equal_and_where_on_strings():
    (e,) = run_node("Equal", {"a": S("x", "y", "z"), "b": S("x", "q", "z")})
    assert e.tolist() == [True, False, True]
    (w,) = run_node("Where", {"c": np.array([True, False]), "a": S("yes", "yes"), "b": S("no", "no")})
    assert w.tolist() == ["yes", "no"]


def test_label_encoder_category_mapper_one_hot_tfidf_with_strings():
    (y,) = run_node("LabelEncoder", {"x": S("a", "b", "d", "a")}, domain=ML, keys_strings=["a", "b", "c"], values_int64s=[0, 1, 2], default_int64=42)
    assert y.tolist() == [0, 1, 42, 0]
    (y,) = run_node("LabelEncoder", {"x": np.array([1, 5, 2], np.int64)}, domain=ML, keys_int64s=[1, 2], values_strings=["one", "two"], default_string="?")
    assert y.tolist() == ["one", "?", "two"]
    (y,) = run_node("LabelEncoder", {"x": S("b", "zz")}, domain=ML, keys_strings=["a", "b"], values_strings=["A", "B"])
    assert y.tolist() == ["B", "_Unused"]
    (y,) = run_node("CategoryMapper", {"x": S("cat", "dog", "cow")}, domain=ML, cats_strings=["cat", "dog"], cats_int64s=[7, 9], default_int64=-5)
    assert y.tolist() == [7, 9, -5]
    (y,) = run_node("CategoryMapper", {"x": np.array([9, 1], np.int64)}, domain=ML, cats_strings=["cat", "dog"], cats_int64s=[7, 9], default_string="none")
    assert y.tolist() == ["dog", "none"]
    (y,) = run_node("OneHotEncoder", {"x": S("b", "c", "x")}, domain=ML, cats_strings=["a", "b", "c"], zeros=1)
    np.testing.assert_array_equal(y, [[0, 1, 0], [0, 0, 1], [0, 0, 0]])
    (y,) = run_node("TfIdfVectorizer", {"x": S("the", "cat", "sat", "the", "cat")}, mode="TF", min_gram_length=1, max_gram_length=2, max_skip_count=0,
                    ngram_counts=[0, 2], ngram_indexes=[0, 1, 2], pool_strings=["the", "sat", "the", "cat"])
    np.testing.assert_array_equal(y, [2, 1, 2])


def test_tokenizer():
    x = S("Absolutely Nothing ", "我 喜欢", shape=(2,))
    (y,) = run_node("Tokenizer", {"x": x}, domain=MS, mark=0, mincharnum=1, pad_value="#", separators=[" "])
    assert y.tolist() == [["Absolutely", "Nothing"], ["我", "喜欢"]]
    (y,) = run_node("Tokenizer", {"x": S("ab c")}, domain=MS, mark=1, mincharnum=1, pad_value="#", separators=[""])
    assert y.tolist() == [["\x02", "a", "b", " ", "c", "\x03"]]
    (y,) = run_node("Tokenizer", {"x": S("a;bb,ccc", "dddd")}, domain=MS, mark=0, mincharnum=2, pad_value="", separators=[";", ","])
    assert y.tolist() == [["bb", "ccc"], ["dddd", ""]]
    (y,) = run_node("Tokenizer", {"x": S("r2d2 and c3po")}, domain=MS, mark=0, mincharnum=1, pad_value="", tokenexp="[a-z]+")
    assert y.tolist() == [["r", "d", "and", "c", "po"]]


def test_string_initializer_through_ort_format():
    from onnxruntime_b200 import ort_format
    vocab = ol.make_tensor("vocab", S("zero", "one", "two"))
    model = ol.make_model(ol.make_graph([ol.make_node("Gather", ["vocab", "idx"], ["y"])], "g", [ol.make_tensor_value_info("idx", T.INT64, ["n"])],
                                        [ol.make_tensor_value_info("y", T.STRING, None)], [vocab]), opset=17)
    buf = ort_format.onnx_to_ort(model)
    back = ort_format.ort_to_onnx(buf)
    assert [s.decode() for s in back.graph.initializers[0].strings] == ["zero", "one", "two"]
    sess = ort.InferenceSession(buf, providers=["CPUExecutionProvider"])
    assert sess.run(None, {"idx": np.array([2, 2, 0], np.int64)})[0].tolist() == ["two", "two", "zero"]


def test_string_tensors_through_ort_values():
    model = graph_model([ol.make_node("StringNormalizer", ["x"], ["y"], case_change_action="UPPER")], [ol.make_tensor_value_info("x", T.STRING, ["n"])],
                        [ol.make_tensor_value_info("y", T.STRING, None)])
    sess = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    v = ort.OrtValue.ortvalue_from_numpy(S("ab", "cd"))
    assert v.data_type() == "tensor(string)" and v.shape() == [2] and v.numpy().tolist() == ["ab", "cd"]
    (out,) = sess.run_with_ort_values(None, {"x": v})
    assert out.data_type() == "tensor(string)" and out.numpy().tolist() == ["AB", "CD"]


def test_strings_through_io_binding():
    """A binding that holds a tensor of strings (input or output) runs by name; bound numeric output buffers are filled."""
    import torch
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    g = ol.make_graph([ol.make_node("StringConcat", ["a", "b"], ["joined"], ), ol.make_node("LabelEncoder", ["a"], ["ids"], domain="ai.onnx.ml",
                                                                                          keys_strings=["x", "y"], values_int64s=[7, 9], default_int64=-1)],
                      "g", [ol.make_tensor_value_info("a", T.STRING, [3]), ol.make_tensor_value_info("b", T.STRING, [3])],
                      [ol.make_tensor_value_info("joined", T.STRING, [3]), ol.make_tensor_value_info("ids", T.INT64, [3])])
    sess = ort.InferenceSession(ol.make_model(g, opset=20, extra_opsets={"ai.onnx.ml": 4}).serialize(), providers=["CPUExecutionProvider"])
    binding = sess.io_binding()
    binding.bind_cpu_input("a", np.array(["x", "q", "y"], dtype=object))
    binding.bind_ortvalue_input("b", ort.OrtValue.ortvalue_from_numpy(np.array(["-1", "-2", "-3"], dtype=object)))
    ids = torch.zeros(3, dtype=torch.int64)
    binding.bind_output("joined")
    binding.bind_torch_output("ids", ids)
    sess.run_with_iobinding(binding)
    joined, ids_out = binding.copy_outputs_to_cpu()
    assert joined.tolist() == ["x-1", "q-2", "y-3"] and ids.tolist() == [7, -1, 9] and ids_out.tolist() == [7, -1, 9]
    assert binding.get_outputs()[0].numpy().tolist() == ["x-1", "q-2", "y-3"]
