"""IOBinding helpers for torch users (counterpart of onnxruntime/python/tools/transformers/io_binding_helper.py):
``TypeHelper`` maps between the session's type strings, numpy and torch dtypes; ``IOBindingHelper`` binds torch tensors;
``CudaSession`` keeps pre-allocated output buffers per shape set and runs with them (the pattern of the reference's
LLM and diffusion pipelines, with CUDA-graph replay when the session options ask for it)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

import onnxruntime_b200 as ort


class TypeHelper:
    _ORT_TO_NUMPY = {"tensor(float)": np.float32, "tensor(float16)": np.float16, "tensor(double)": np.float64, "tensor(int64)": np.int64,
                     "tensor(int32)": np.int32, "tensor(int8)": np.int8, "tensor(uint8)": np.uint8, "tensor(bool)": np.bool_,
                     "tensor(int16)": np.int16, "tensor(uint16)": np.uint16}
    _ORT_TO_TORCH = {"tensor(float)": torch.float32, "tensor(float16)": torch.float16, "tensor(double)": torch.float64,
                     "tensor(int64)": torch.int64, "tensor(int32)": torch.int32, "tensor(int8)": torch.int8, "tensor(uint8)": torch.uint8,
                     "tensor(bool)": torch.bool, "tensor(bfloat16)": torch.bfloat16, "tensor(int16)": torch.int16}

    @staticmethod
    def get_input_type(sess: "ort.InferenceSession", name: str) -> str:
        for i in sess.get_inputs():
            if i.name == name:
                return i.type
        raise ValueError(f"input name {name} not found")

    @staticmethod
    def get_output_type(sess: "ort.InferenceSession", name: str) -> str:
        for o in sess.get_outputs():
            if o.name == name:
                return o.type
        raise ValueError(f"output name {name} not found")

    @staticmethod
    def ort_type_to_numpy_type(ort_type: str):
        if ort_type not in TypeHelper._ORT_TO_NUMPY:
            raise ValueError(f"{ort_type} not found in map")
        return TypeHelper._ORT_TO_NUMPY[ort_type]

    @staticmethod
    def ort_type_to_torch_type(ort_type: str):
        if ort_type not in TypeHelper._ORT_TO_TORCH:
            raise ValueError(f"{ort_type} not found in map")
        return TypeHelper._ORT_TO_TORCH[ort_type]

    @staticmethod
    def numpy_type_to_torch_type(numpy_type):
        return torch.from_numpy(np.zeros(1, dtype=numpy_type)).dtype

    @staticmethod
    def torch_type_to_numpy_type(torch_type):
        return torch.zeros(1, dtype=torch_type).numpy().dtype.type

    @staticmethod
    def get_io_numpy_type_map(sess: "ort.InferenceSession") -> Dict[str, type]:
        return {a.name: TypeHelper.ort_type_to_numpy_type(a.type) for a in list(sess.get_inputs()) + list(sess.get_outputs())
                if a.type in TypeHelper._ORT_TO_NUMPY}

    @staticmethod
    def get_io_torch_type_map(sess: "ort.InferenceSession") -> Dict[str, torch.dtype]:
        return {a.name: TypeHelper.ort_type_to_torch_type(a.type) for a in list(sess.get_inputs()) + list(sess.get_outputs())
                if a.type in TypeHelper._ORT_TO_TORCH}


class IOBindingHelper:
    @staticmethod
    def get_output_buffers(sess: "ort.InferenceSession", output_shapes: Dict[str, Sequence[int]], device) -> Dict[str, torch.Tensor]:
        types = TypeHelper.get_io_torch_type_map(sess)
        return {n: torch.empty(tuple(int(d) for d in shape), dtype=types[n], device=device) for n, shape in output_shapes.items()}

    @staticmethod
    def prepare_io_binding(sess: "ort.InferenceSession", inputs: Dict[str, torch.Tensor], output_buffers: Dict[str, torch.Tensor]):
        binding = sess.io_binding()
        for name, t in inputs.items():
            binding.bind_torch_input(name, t.contiguous())
        for name, t in output_buffers.items():
            binding.bind_torch_output(name, t)
        return binding


class CudaSession:
    """Session + reusable output buffers; `infer` binds the feeds, runs and returns the buffers (no host copies)."""

    def __init__(self, sess: "ort.InferenceSession", device: torch.device, enable_cuda_graph: bool = False):
        self.sess, self.device, self.enable_cuda_graph = sess, torch.device(device), enable_cuda_graph
        self.input_names = [i.name for i in sess.get_inputs()]
        self.output_names = [o.name for o in sess.get_outputs()]
        self.io_name_to_torch_type = TypeHelper.get_io_torch_type_map(sess)
        self.output_tensors: Dict[str, torch.Tensor] = {}
        self.input_tensors: Dict[str, torch.Tensor] = {}
        self.binding = sess.io_binding()

    def allocate_buffers(self, shape_dict: Dict[str, Sequence[int]]) -> None:
        """Buffers for every named input / output in `shape_dict`; inputs get buffers only when CUDA graphs need fixed addresses."""
        for name, shape in shape_dict.items():
            shape = tuple(int(d) for d in shape)
            if name in self.output_names:
                if name not in self.output_tensors or tuple(self.output_tensors[name].shape) != shape:
                    self.output_tensors[name] = torch.empty(shape, dtype=self.io_name_to_torch_type[name], device=self.device)
                    self.binding.bind_torch_output(name, self.output_tensors[name])
            elif name in self.input_names and self.enable_cuda_graph:
                if name not in self.input_tensors or tuple(self.input_tensors[name].shape) != shape:
                    self.input_tensors[name] = torch.empty(shape, dtype=self.io_name_to_torch_type[name], device=self.device)
                    self.binding.bind_torch_input(name, self.input_tensors[name])

    def infer(self, feed_dict: Dict[str, torch.Tensor], run_options: Optional["ort.RunOptions"] = None, synchronize: bool = True) -> Dict[str, torch.Tensor]:
        for name, t in feed_dict.items():
            if name in self.input_tensors:
                self.input_tensors[name].copy_(t)       # fixed address: copy into the bound buffer
            else:
                self.binding.bind_torch_input(name, t.to(self.device).contiguous())
        for name in self.output_names:
            if name not in self.output_tensors:
                self.binding.bind_output(name, self.device.type, self.device.index or 0)
        self.sess.run_with_iobinding(self.binding, run_options)
        if synchronize:
            self.binding.synchronize_outputs()
        if len(self.output_tensors) == len(self.output_names):
            return self.output_tensors
        outs = self.binding.get_outputs()
        return {n: self.output_tensors.get(n, o.as_torch()) for n, o in zip(self.output_names, outs)}
