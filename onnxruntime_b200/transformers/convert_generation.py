"""Wrap exported decoder (and encoder) graphs into one model whose single node is a generation operator.

Counterpart of the reference's ``python -m onnxruntime.transformers.convert_generation``
(onnxruntime/python/tools/transformers/convert_generation.py): the decoder ONNX becomes the ``decoder`` body of a
``com.microsoft`` BeamSearch / GreedySearch / Sampling node (plus ``encoder`` for T5- and Whisper-style models), and
the search parameters become graph inputs.

    python -m onnxruntime_b200.transformers.convert_generation --decoder_onnx decoder.onnx --output gpt2_beam.onnx \\
        --num_beams_op beam --eos_token_id 50256 --pad_token_id 50256 --no_repeat_ngram_size 3

Body contracts: see the generation kernel (csrc/core/kernels_controlflow.cc).  GPT form: the decoder takes
``input_ids, position_ids, attention_mask, past_0 ...`` and returns ``logits, present_0 ...``.
"""
from __future__ import annotations

import argparse
import sys
from typing import List, Optional

from .. import onnx_lite as ol

T = ol.TensorProto
OPS = {"beam": "BeamSearch", "greedy": "GreedySearch", "sampling": "Sampling", "whisper": "WhisperBeamSearch"}


def convert(decoder: ol.Model, op: str = "beam", encoder: Optional[ol.Model] = None, model_type: int = 0, eos_token_id: int = -1,
            pad_token_id: int = 0, decoder_start_token_id: int = 0, no_repeat_ngram_size: int = 0, early_stopping: bool = False,
            vocab_mask: bool = False, prefix_vocab_mask: bool = False, attention_mask: bool = True, **sampling_attrs) -> ol.Model:
    op_type = OPS[op]
    beam = op_type in ("BeamSearch", "WhisperBeamSearch")
    if op_type == "WhisperBeamSearch":
        model_type = 2
    if model_type != 0 and encoder is None:
        raise ValueError("encoder-decoder models need the encoder graph")
    first = ("input_features", T.FLOAT, ["batch", "features", "frames"]) if model_type == 2 else ("input_ids", T.INT32, ["batch", "sequence"])
    names: List[str] = [first[0], "max_length", "min_length"]
    infos = [ol.make_tensor_value_info(*first), ol.make_tensor_value_info("max_length", T.INT32, [1]),
             ol.make_tensor_value_info("min_length", T.INT32, [1])]
    if beam:
        names += ["num_beams", "num_return_sequences", "length_penalty"]
        infos += [ol.make_tensor_value_info("num_beams", T.INT32, [1]), ol.make_tensor_value_info("num_return_sequences", T.INT32, [1]),
                  ol.make_tensor_value_info("length_penalty", T.FLOAT, [1])]
    names.append("repetition_penalty")
    infos.append(ol.make_tensor_value_info("repetition_penalty", T.FLOAT, [1]))
    for flag, name, shape in ((vocab_mask, "vocab_mask", ["vocab"]), (prefix_vocab_mask, "prefix_vocab_mask", ["batch", "vocab"]),
                              (attention_mask and model_type != 2, "attention_mask", ["batch", "sequence"])):
        names.append(name if flag else "")
        if flag:
            infos.append(ol.make_tensor_value_info(name, T.INT32, shape))
    while names and names[-1] == "":
        names.pop()
    outputs = ["sequences"] + (["sequences_scores"] if beam else [])
    attrs = dict(decoder=decoder.graph, model_type=model_type, eos_token_id=eos_token_id, pad_token_id=pad_token_id,
                 no_repeat_ngram_size=no_repeat_ngram_size, early_stopping=int(early_stopping))
    if encoder is not None:
        attrs.update(encoder=encoder.graph, decoder_start_token_id=decoder_start_token_id)
    if op_type == "Sampling":
        attrs.update({k: v for k, v in sampling_attrs.items() if v is not None})
    node = ol.make_node(op_type, names, outputs, domain="com.microsoft", name=f"{op_type}_0", **attrs)
    out_infos = [ol.make_tensor_value_info("sequences", T.INT32, ["batch", "num_return_sequences", "max_length"] if beam else ["batch", "max_length"])]
    if beam:
        out_infos.append(ol.make_tensor_value_info("sequences_scores", T.FLOAT, ["batch", "num_return_sequences"]))
    opset = max(decoder.opset_imports.get("", 17), 13)
    return ol.make_model(ol.make_graph([node], f"{op_type} wrapper", infos, out_infos), opset=opset)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--decoder_onnx", required=True)
    ap.add_argument("--encoder_onnx", default=None)
    ap.add_argument("--output", required=True)
    ap.add_argument("--num_beams_op", default="beam", choices=sorted(OPS), help="which generation operator drives the decoder")
    ap.add_argument("--model_type", type=int, default=0, help="0 GPT, 1 T5, 2 Whisper")
    ap.add_argument("--eos_token_id", type=int, default=-1)
    ap.add_argument("--pad_token_id", type=int, default=0)
    ap.add_argument("--decoder_start_token_id", type=int, default=0)
    ap.add_argument("--no_repeat_ngram_size", type=int, default=0)
    ap.add_argument("--early_stopping", action="store_true")
    ap.add_argument("--vocab_mask", action="store_true")
    ap.add_argument("--prefix_vocab_mask", action="store_true")
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top_p", type=float, default=None)
    ap.add_argument("--seed", type=int, default=None)
    a = ap.parse_args(argv)
    model = convert(ol.load_model(a.decoder_onnx), a.num_beams_op, ol.load_model(a.encoder_onnx) if a.encoder_onnx else None, a.model_type,
                    a.eos_token_id, a.pad_token_id, a.decoder_start_token_id, a.no_repeat_ngram_size, a.early_stopping, a.vocab_mask,
                    a.prefix_vocab_mask, temperature=a.temperature, top_p=a.top_p, seed=a.seed)
    with open(a.output, "wb") as f:
        f.write(model.serialize())
    print(f"wrote {a.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
