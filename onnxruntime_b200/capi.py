"""Python API shell over the native runtime (``_core``).

Keeps the user-facing contract of the reference's Python package
(onnxruntime/python/onnxruntime_inference_collection.py: ``InferenceSession``
:469, ``Session.run`` :308, ``IOBinding`` :888, ``OrtValue`` :1022,
``OrtDevice`` :1362): ``InferenceSession(path_or_bytes, sess_options, providers,
provider_options).run(output_names, feeds)``, ``SessionOptions`` / ``RunOptions``
properties, ``io_binding()`` with device-resident inputs and outputs, and the
exception classes.  Tensors are ``torch.Tensor`` underneath, so an ``OrtValue``
can wrap CUDA memory, bf16 and fp8 without a copy.
"""
from __future__ import annotations

import os
import threading
from struct import error as struct_error
from enum import IntEnum
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _core as C

__all__ = [
    "AdapterFormat", "LoraAdapter", "register_custom_op",
    "InferenceSession", "SessionOptions", "RunOptions", "IOBinding", "OrtValue", "OrtDevice", "NodeArg",
    "ModelMetadata", "GraphOptimizationLevel", "ExecutionMode", "ExecutionOrder", "get_available_providers",
    "get_all_providers", "get_device", "set_default_logger_severity", "set_default_logger_verbosity", "set_log_sink",
    "ModelCompiler", "OrtValueVector", "SparseTensor", "OrtEpDevice", "OrtExecutionProviderDevicePolicy", "get_ep_devices",
    "get_version_string", "get_build_info", "has_collective_ops", "set_seed", "enable_telemetry_events", "disable_telemetry_events",
    "ModelLoadCanceled", "ModelRequiresCompilation", "NotFound",
]


# ------------------------------------------------------------------ exceptions
class OrtException(Exception):
    """Base of the runtime's exceptions."""


class Fail(OrtException, RuntimeError): pass
class InvalidArgument(OrtException, ValueError): pass
class NoSuchFile(OrtException, FileNotFoundError): pass
class NoModel(OrtException): pass
class EngineError(OrtException): pass
class RuntimeException(OrtException, RuntimeError): pass
class InvalidProtobuf(OrtException): pass
class ModelLoaded(OrtException): pass
class NotImplemented(OrtException, NotImplementedError): pass  # noqa: A001 (name kept for API parity)
class InvalidGraph(OrtException): pass
class EPFail(OrtException): pass
class ModelLoadCanceled(OrtException): pass
class ModelRequiresCompilation(OrtException): pass
class NotFound(OrtException): pass


_CODE_NAMES = {1: "FAIL", 2: "INVALID_ARGUMENT", 3: "NO_SUCHFILE", 4: "NO_MODEL", 5: "ENGINE_ERROR",
               6: "RUNTIME_EXCEPTION", 7: "INVALID_PROTOBUF", 8: "MODEL_LOADED", 9: "NOT_IMPLEMENTED",
               10: "INVALID_GRAPH", 11: "EP_FAIL", 12: "MODEL_LOAD_CANCELED", 13: "MODEL_REQUIRES_COMPILATION",
               14: "NOT_FOUND"}
_CODE_CLASSES = {1: Fail, 2: InvalidArgument, 3: NoSuchFile, 4: NoModel, 5: EngineError, 6: RuntimeException,
                 7: InvalidProtobuf, 8: ModelLoaded, 9: NotImplemented, 10: InvalidGraph, 11: EPFail,
                 12: ModelLoadCanceled, 13: ModelRequiresCompilation, 14: NotFound}


def _make_error(code: int, message: str) -> Exception:
    cls = _CODE_CLASSES.get(code, Fail)
    return cls(f"[ONNXRuntimeError] : {code} : {_CODE_NAMES.get(code, 'FAIL')} : {message}")


C.set_error_factory(_make_error)


# ----------------------------------------------------------------------- enums
class GraphOptimizationLevel(IntEnum):
    ORT_DISABLE_ALL = 0
    ORT_ENABLE_BASIC = 1
    ORT_ENABLE_EXTENDED = 2
    ORT_ENABLE_LAYOUT = 3
    ORT_ENABLE_ALL = 99


class ExecutionMode(IntEnum):
    ORT_SEQUENTIAL = 0
    ORT_PARALLEL = 1


class OrtExecutionProviderDevicePolicy(IntEnum):
    DEFAULT = 0
    PREFER_CPU = 1
    PREFER_NPU = 2
    PREFER_GPU = 3
    MAX_PERFORMANCE = 4
    MAX_EFFICIENCY = 5
    MIN_OVERALL_POWER = 6


class ExecutionOrder(IntEnum):
    DEFAULT = 0
    PRIORITY_BASED = 1
    MEMORY_EFFICIENT = 2


_ALL_PROVIDERS = ["CUDAExecutionProvider", "CPUExecutionProvider"]
_default_logger_severity = 2
_default_logger_verbosity = 0


def get_all_providers() -> List[str]:
    return list(_ALL_PROVIDERS)


def get_available_providers() -> List[str]:
    out = []
    if torch.cuda.is_available():
        out.append("CUDAExecutionProvider")
    out.append("CPUExecutionProvider")
    return out


def get_device() -> str:
    return "GPU" if torch.cuda.is_available() else "CPU"


def get_version_string() -> str:
    from . import __version__
    return __version__


def get_build_info() -> str:
    return (f"onnxruntime_b200 {get_version_string()}, sm_100a kernels, torch {torch.__version__}, "
            f"cuda {torch.version.cuda or 'none'}")


def has_collective_ops() -> bool:
    """AllReduce / AllGather / AllToAll / ShardedMoE / Distributed* are always part of the build."""
    return True


def set_seed(seed: int) -> None:
    """Seed of the random operators (RandomNormal, Multinomial, Dropout in training mode, Sampling ...)."""
    torch.manual_seed(int(seed))


def enable_telemetry_events() -> None:
    """Kept for API parity: this runtime collects no telemetry."""


def disable_telemetry_events() -> None:
    """Kept for API parity: this runtime collects no telemetry."""


class OrtEpDevice:
    """One (execution provider, hardware device) pair, as ``get_ep_devices`` lists them."""

    def __init__(self, ep_name: str, device_type: str, device_id: int, vendor: str, metadata: Dict[str, str]):
        self.ep_name, self.ep_vendor = ep_name, "onnxruntime_b200"
        self.device = OrtDevice(device_type, device_id)
        self.ep_metadata, self.ep_options = dict(metadata), {}
        self.device_vendor = vendor

    def __repr__(self) -> str:
        return f"OrtEpDevice({self.ep_name}, {self.device.device_type()}:{self.device.device_id()})"


def get_ep_devices() -> List["OrtEpDevice"]:
    out = [OrtEpDevice("CPUExecutionProvider", "cpu", 0, "host", {})]
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            out.append(OrtEpDevice("CUDAExecutionProvider", "cuda", i, "NVIDIA",
                                   {"name": p.name, "compute_capability": f"{p.major}.{p.minor}", "memory_bytes": str(p.total_memory)}))
    return out


def set_default_logger_severity(severity: int) -> None:
    global _default_logger_severity
    if not 0 <= severity <= 4:
        raise InvalidArgument("severity must be in [0, 4]")
    _default_logger_severity = severity
    C.set_default_logger_severity(severity)


def set_default_logger_verbosity(verbosity: int) -> None:
    global _default_logger_verbosity
    _default_logger_verbosity = verbosity
    C.set_default_logger_verbosity(verbosity)


def set_log_sink(sink) -> None:
    """Route log lines to ``sink(severity, logger_id, line)`` instead of stderr; ``None`` restores stderr."""
    C.set_log_sink(sink)


# ------------------------------------------------------------------ type names
_TORCH_TO_TYPESTR = {
    torch.float32: "tensor(float)", torch.float16: "tensor(float16)", torch.bfloat16: "tensor(bfloat16)",
    torch.float64: "tensor(double)", torch.int64: "tensor(int64)", torch.int32: "tensor(int32)",
    torch.int16: "tensor(int16)", torch.int8: "tensor(int8)", torch.uint8: "tensor(uint8)", torch.bool: "tensor(bool)",
    torch.uint16: "tensor(uint16)", torch.uint32: "tensor(uint32)", torch.uint64: "tensor(uint64)",
    torch.float8_e4m3fn: "tensor(float8e4m3fn)", torch.float8_e5m2: "tensor(float8e5m2)",
}
_ONNX_ELEM_TO_TORCH = {
    1: torch.float32, 2: torch.uint8, 3: torch.int8, 4: torch.uint16, 5: torch.int16, 6: torch.int32, 7: torch.int64,
    9: torch.bool, 10: torch.float16, 11: torch.float64, 12: torch.uint32, 13: torch.uint64, 16: torch.bfloat16,
    17: torch.float8_e4m3fn, 19: torch.float8_e5m2,
}


def _is_ort_format(buf: bytes) -> bool:
    return len(buf) >= 8 and bytes(buf[4:8]) == b"ORTM"


class _StringTensor:
    """A tensor of strings on its way into or out of the runtime (which carries ids of its string table)."""

    def __init__(self, strings: List[str], shape: Sequence[int]):
        self.strings, self.shape = list(strings), tuple(int(d) for d in shape)

    def numpy(self) -> np.ndarray:
        out = np.empty(len(self.strings), dtype=object)
        out[:] = self.strings
        return out.reshape(self.shape)


def _is_string_array(value: Any) -> bool:
    if isinstance(value, np.ndarray):
        if value.dtype.kind in "US":
            return True
        return value.dtype.kind == "O" and value.size > 0 and isinstance(value.reshape(-1)[0], (str, bytes))
    if isinstance(value, (str, bytes)):
        return True
    return isinstance(value, (list, tuple)) and len(value) > 0 and isinstance(np.asarray(value, dtype=object).reshape(-1)[0], (str, bytes))


def _to_torch(value: Any) -> torch.Tensor:
    if isinstance(value, SparseTensor):
        return value._t.to_dense()
    if isinstance(value, OrtValue):
        value = value._tensor
    if isinstance(value, _StringTensor):
        return value
    if isinstance(value, torch.Tensor):
        return value.to_dense() if value.layout != torch.strided else value
    if isinstance(value, dict):      # a map-typed input (ai.onnx.ml CastMap / DictVectorizer): converted by the native layer
        return value
    if _is_string_array(value):
        arr = np.asarray(value, dtype=object)
        flat = [s.decode("utf-8") if isinstance(s, bytes) else str(s) for s in arr.reshape(-1)]
        return _StringTensor(flat, arr.shape)
    if isinstance(value, np.ndarray):
        if not value.flags.c_contiguous:
            value = np.ascontiguousarray(value)
        if not value.flags.writeable:
            value = value.copy()
        return torch.from_numpy(value)
    if isinstance(value, (list, tuple)) and value and isinstance(value[0], (np.ndarray, torch.Tensor, OrtValue)):
        return [_to_torch(v) for v in value]  # sequence input
    return torch.as_tensor(np.asarray(value))


def _to_numpy(t: Any) -> Any:
    if t is None:
        return None
    if isinstance(t, dict):        # a row of a ZipMap output
        return t
    if isinstance(t, list):
        return [_to_numpy(x) for x in t]
    if isinstance(t, tuple) and len(t) == 3 and t[0] == "__strings__":
        return _StringTensor(t[1], t[2]).numpy()
    t = t.detach()
    if t.is_cuda:
        t = t.cpu()
    if t.dtype in (torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2):
        t = t.float()  # numpy has no such dtype
    return t.numpy()


# --------------------------------------------------------------------- OrtDevice
class OrtDevice:
    """Device descriptor ("cpu" or "cuda", device id)."""

    def __init__(self, device_type: str = "cpu", device_id: int = 0):
        self._type = device_type.lower()
        self._id = device_id

    @staticmethod
    def cpu() -> str:
        return "cpu"

    @staticmethod
    def cuda() -> str:
        return "cuda"

    @staticmethod
    def make(ort_device_name: str, device_id: int) -> "OrtDevice":
        return OrtDevice(ort_device_name, device_id)

    def device_id(self) -> int:
        return self._id

    def device_type(self) -> str:
        return self._type

    def _torch(self) -> torch.device:
        return torch.device("cuda", self._id) if self._type == "cuda" else torch.device("cpu")


# ---------------------------------------------------------------------- OrtValue
class OrtValue:
    """A tensor owned by (or shared with) the runtime; wraps a ``torch.Tensor``."""

    def __init__(self, tensor: torch.Tensor):
        self._tensor = tensor

    @staticmethod
    def ortvalue_from_numpy(numpy_obj: np.ndarray, device_type: str = "cpu", device_id: int = 0) -> "OrtValue":
        t = _to_torch(numpy_obj)
        if device_type.lower() == "cuda":
            t = t.to(torch.device("cuda", device_id))
        return OrtValue(t)

    @staticmethod
    def ortvalue_from_shape_and_type(shape: Sequence[int], element_type=np.float32, device_type: str = "cpu",
                                     device_id: int = 0) -> "OrtValue":
        if isinstance(element_type, int):
            dt = _ONNX_ELEM_TO_TORCH[element_type]
        elif isinstance(element_type, torch.dtype):
            dt = element_type
        else:
            dt = torch.from_numpy(np.zeros((), dtype=element_type)).dtype
        dev = torch.device("cuda", device_id) if device_type.lower() == "cuda" else torch.device("cpu")
        return OrtValue(torch.empty(tuple(shape), dtype=dt, device=dev))

    @staticmethod
    def ortvalue_from_torch(tensor: torch.Tensor) -> "OrtValue":
        return OrtValue(tensor)

    @staticmethod
    def from_dlpack(data, is_bool_tensor: bool = False) -> "OrtValue":
        t = torch.utils.dlpack.from_dlpack(data)
        if is_bool_tensor:
            t = t.view(torch.bool)
        return OrtValue(t)

    def __dlpack__(self, stream=None):
        return self._tensor.__dlpack__() if stream is None else self._tensor.__dlpack__(stream=stream)

    def __dlpack_device__(self):
        return self._tensor.__dlpack_device__()

    def to_dlpack(self):
        return torch.utils.dlpack.to_dlpack(self._tensor)

    def as_torch(self) -> torch.Tensor:
        return self._tensor

    def data_ptr(self) -> int:
        return self._tensor.data_ptr()

    def device_name(self) -> str:
        return "cuda" if getattr(self._tensor, "is_cuda", False) else "cpu"

    def shape(self) -> List[int]:
        return list(self._tensor.shape)

    def data_type(self) -> str:
        if isinstance(self._tensor, _StringTensor):
            return "tensor(string)"
        return _TORCH_TO_TYPESTR.get(self._tensor.dtype, "tensor(unknown)")

    def element_type(self) -> int:
        if isinstance(self._tensor, _StringTensor):
            return 8
        for k, v in _ONNX_ELEM_TO_TORCH.items():
            if v == self._tensor.dtype:
                return k
        return 0

    def has_value(self) -> bool:
        return self._tensor is not None

    def is_tensor(self) -> bool:
        return True

    def is_sparse_tensor(self) -> bool:
        return bool(getattr(self._tensor, "is_sparse", False) or getattr(self._tensor, "is_sparse_csr", False))

    @staticmethod
    def ort_value_from_sparse_tensor(sparse_tensor: "SparseTensor") -> "OrtValue":
        return OrtValue(sparse_tensor._t)

    def as_sparse_tensor(self) -> "SparseTensor":
        if not self.is_sparse_tensor():
            raise InvalidArgument("this OrtValue does not hold a sparse tensor")
        return SparseTensor(self._tensor)

    def is_tensor_sequence(self) -> bool:
        return False

    def numpy(self) -> np.ndarray:
        if isinstance(self._tensor, _StringTensor):
            return self._tensor.numpy()
        return _to_numpy(self._tensor)

    def update_inplace(self, np_arr: np.ndarray) -> None:
        self._tensor.copy_(_to_torch(np_arr))


class OrtValueVector:
    """A growable list of OrtValues (the reference's ``OrtValueVector``)."""

    def __init__(self, values: Optional[Sequence["OrtValue"]] = None):
        self._v: List[OrtValue] = list(values or [])

    def push_back(self, value) -> None:
        self._v.append(value if isinstance(value, OrtValue) else OrtValue(_to_torch(value)))

    def push_back_batch(self, tensors: Sequence[Any], *_ignored) -> None:
        for t in tensors:
            self.push_back(t)

    def reserve(self, n: int) -> None:
        pass

    def shrink_to_fit(self) -> None:
        pass

    def clear(self) -> None:
        self._v.clear()

    def __len__(self) -> int:
        return len(self._v)

    def __getitem__(self, i) -> "OrtValue":
        return self._v[i]

    def __iter__(self):
        return iter(self._v)

    def dlpack_at(self, i: int):
        return self._v[i].to_dlpack()

    def to_dlpacks(self, to_tensor=None) -> List[Any]:
        caps = [v.to_dlpack() for v in self._v]
        return caps if to_tensor is None else [to_tensor(c) for c in caps]

    def bool_tensor_indices(self) -> List[int]:
        return [i for i, v in enumerate(self._v) if v._tensor.dtype == torch.bool]

    def element_type_at(self, i: int) -> int:
        return self._v[i].element_type()


class _SparseView:
    def __init__(self, **parts):
        self._parts = parts

    def __getattr__(self, name):
        if name in self._parts:
            return lambda: self._parts[name]
        raise AttributeError(name)


class SparseTensor:
    """COO / CSR sparse tensors (the reference's ``SparseTensor``), held as torch sparse tensors.  The runtime's kernels are
    dense: a sparse feed or initializer is expanded when it enters a session."""

    def __init__(self, t: torch.Tensor):
        self._t = t

    @staticmethod
    def sparse_coo_from_numpy(dense_shape, values: np.ndarray, coo_indices: np.ndarray, ort_device: Optional[OrtDevice] = None) -> "SparseTensor":
        shape = [int(d) for d in dense_shape]
        idx = torch.as_tensor(np.asarray(coo_indices, dtype=np.int64))
        if idx.dim() == 1:      # linear indices into the flattened tensor
            idx = torch.stack(torch.unravel_index(idx, shape)) if shape else idx.reshape(0, -1)
        else:                   # [nnz, rank] coordinates
            idx = idx.t().contiguous()
        t = torch.sparse_coo_tensor(idx, torch.as_tensor(np.asarray(values)), shape).coalesce()
        return SparseTensor(t.to(ort_device._torch()) if ort_device is not None else t)

    @staticmethod
    def sparse_csr_from_numpy(dense_shape, values: np.ndarray, inner_indices: np.ndarray, outer_indices: np.ndarray,
                              ort_device: Optional[OrtDevice] = None) -> "SparseTensor":
        t = torch.sparse_csr_tensor(torch.as_tensor(np.asarray(outer_indices, dtype=np.int64)), torch.as_tensor(np.asarray(inner_indices, dtype=np.int64)),
                                    torch.as_tensor(np.asarray(values)), [int(d) for d in dense_shape])
        return SparseTensor(t.to(ort_device._torch()) if ort_device is not None else t)

    def values(self) -> np.ndarray:
        return self._t.values().cpu().numpy()

    def as_coo_view(self):
        if self._t.layout != torch.sparse_coo:
            raise InvalidArgument("not a COO tensor")
        return _SparseView(indices=self._t.indices().t().contiguous().cpu().numpy())

    def as_csrc_view(self):
        if self._t.layout != torch.sparse_csr:
            raise InvalidArgument("not a CSR tensor")
        return _SparseView(inner=self._t.col_indices().cpu().numpy(), outer=self._t.crow_indices().cpu().numpy())

    def to_cuda(self, ort_device: OrtDevice) -> "SparseTensor":
        return SparseTensor(self._t.to(ort_device._torch()))

    def to_dense(self) -> np.ndarray:
        return self._t.to_dense().cpu().numpy()

    def format(self) -> str:
        return "COO" if self._t.layout == torch.sparse_coo else "CSR"

    def dense_shape(self) -> List[int]:
        return list(self._t.shape)

    def data_type(self) -> str:
        return f"sparse_tensor({_TORCH_TYPE_NAMES.get(self._t.dtype, str(self._t.dtype))})"

    def device_name(self) -> str:
        return "Cuda" if self._t.is_cuda else "Cpu"


_TORCH_TYPE_NAMES = {torch.float32: "float", torch.float16: "float16", torch.float64: "double", torch.int64: "int64", torch.int32: "int32",
                     torch.int8: "int8", torch.uint8: "uint8", torch.bool: "bool", torch.bfloat16: "bfloat16"}


class NodeArg:
    """Name, type string and shape of a model input or output."""

    def __init__(self, meta):
        self.name = meta.name
        self.type = meta.type
        if meta.has_shape:
            self.shape = [d if d >= 0 else (s if s else None) for d, s in zip(meta.shape, meta.sym)]
        else:
            self.shape = None

    def __repr__(self) -> str:
        return f"NodeArg(name='{self.name}', type='{self.type}', shape={self.shape})"


class ModelMetadata:
    def __init__(self, d: Dict[str, Any]):
        self.producer_name = d["producer_name"]
        self.graph_name = d["graph_name"]
        self.domain = d["domain"]
        self.description = d["description"]
        self.graph_description = d["graph_description"]
        self.version = d["version"]
        self.custom_metadata_map = dict(d["custom_metadata_map"])


# ----------------------------------------------------------------- SessionOptions
class SessionOptions:
    """Session configuration; property names follow the reference's pybind ``SessionOptions``."""

    _FIELDS = ("enable_cpu_mem_arena", "enable_mem_pattern", "enable_mem_reuse", "enable_profiling",
               "profile_file_prefix", "optimized_model_filepath", "logid", "log_severity_level", "log_verbosity_level",
               "intra_op_num_threads", "inter_op_num_threads", "use_deterministic_compute", "use_per_session_threads")

    def __init__(self):
        object.__setattr__(self, "_c", C.SessionOptions())
        object.__setattr__(self, "_custom_op_libraries", [])
        object.__setattr__(self, "_keepalive", [])

    def __getattr__(self, name):
        if name in SessionOptions._FIELDS:
            return getattr(self._c, name)
        raise AttributeError(name)

    def __setattr__(self, name, value):
        if name in SessionOptions._FIELDS:
            setattr(self._c, name, value)
        elif name in ("execution_mode", "execution_order", "graph_optimization_level"):
            setattr(self._c, name, int(value))
        else:
            raise AttributeError(f"SessionOptions has no attribute '{name}'")

    @property
    def execution_mode(self) -> ExecutionMode:
        return ExecutionMode(self._c.execution_mode)

    @property
    def execution_order(self) -> ExecutionOrder:
        return ExecutionOrder(self._c.execution_order)

    @property
    def graph_optimization_level(self) -> GraphOptimizationLevel:
        return GraphOptimizationLevel(self._c.graph_optimization_level)

    def add_session_config_entry(self, key: str, value: str) -> None:
        self._c.add_config(key, str(value))

    def get_session_config_entry(self, key: str) -> str:
        v = self._c.get_config(key)
        if v is None:
            raise RuntimeException(f"Session config entry '{key}' was not found.")
        return v

    def add_free_dimension_override_by_name(self, name: str, value: int) -> None:
        self._c.add_free_dim_by_name(name, int(value))

    def add_free_dimension_override_by_denotation(self, denotation: str, value: int) -> None:
        self._c.add_free_dim_by_denotation(denotation, int(value))

    def add_initializer(self, name: str, ort_value: OrtValue) -> None:
        self._c.add_initializer(name, _to_torch(ort_value))

    def add_external_initializers(self, names: Sequence[str], ort_values: Sequence[Any]) -> None:
        if len(names) != len(ort_values):
            raise InvalidArgument("names and ort_values differ in length")
        for n, v in zip(names, ort_values):
            self._c.add_external_initializer(n, _to_torch(v))

    def add_external_initializers_from_files_in_memory(self, names: Sequence[str], buffers: Sequence[Any], lengths: Sequence[int]) -> None:
        """External-data FILES handed over as memory: `names` are the file names the model's initializers point to.  The
        bytes are kept for the model load, which reads the initializers' (offset, length) ranges from them."""
        if not (len(names) == len(buffers) == len(lengths)):
            raise InvalidArgument("names, buffers and lengths differ in length")
        files = dict(getattr(self, "_external_files", {}))
        for n, b, ln in zip(names, buffers, lengths):
            files[os.fspath(n)] = bytes(memoryview(b)[:int(ln)])
        object.__setattr__(self, "_external_files", files)

    def add_provider_for_devices(self, ep_devices: Sequence["OrtEpDevice"], provider_options: Optional[Dict[str, str]] = None) -> None:
        """Pin the session to the provider of the given devices (all of one provider)."""
        names = {d.ep_name for d in ep_devices}
        if len(names) != 1:
            raise InvalidArgument("add_provider_for_devices needs devices of exactly one execution provider")
        opts = dict(provider_options or {})
        dev = ep_devices[0].device
        if dev.device_type() == "cuda":
            opts.setdefault("device_id", str(dev.device_id()))
        chosen = list(getattr(self, "_providers_for_devices", []))
        chosen.append((names.pop(), opts))
        object.__setattr__(self, "_providers_for_devices", chosen)

    def add_provider(self, name: str, provider_options: Optional[Dict[str, str]] = None) -> None:
        chosen = list(getattr(self, "_providers_for_devices", []))
        chosen.append((name, dict(provider_options or {})))
        object.__setattr__(self, "_providers_for_devices", chosen)

    def set_provider_selection_policy(self, policy) -> None:
        """Automatic provider selection: PREFER_GPU / MAX_PERFORMANCE pick the CUDA provider when a GPU is there,
        PREFER_CPU / MIN_OVERALL_POWER the CPU provider; DEFAULT leaves the choice to the `providers` argument."""
        object.__setattr__(self, "_selection_policy", OrtExecutionProviderDevicePolicy(int(policy)))

    def set_provider_selection_policy_delegate(self, delegate) -> None:
        """delegate(ep_devices, model_metadata, runtime_metadata, max_selections) -> the devices to use."""
        object.__setattr__(self, "_selection_delegate", delegate)

    def set_load_cancellation_flag(self, value: bool) -> None:
        """A session created while the flag is set fails with ModelLoadCanceled."""
        object.__setattr__(self, "_load_cancelled", bool(value))

    def register_custom_ops_library(self, path: str) -> None:
        if not os.path.exists(path):
            raise NoSuchFile(f"custom op library {path} not found")
        # the library exports ortb200_register_custom_ops (csrc/core/custom_op_api.h); its operators join the
        # kernel registry of the process, as the reference's RegisterCustomOps entry point does per session
        C.load_custom_op_library(os.fspath(path))


class RunOptions:
    def __init__(self):
        self._c = C.RunOptions()
        self._adapters: List["LoraAdapter"] = []

    def add_active_adapter(self, adapter: "LoraAdapter") -> None:
        """The adapter's parameters are fed as extra inputs of every run made with these options (they override the
        model's same-named optional inputs / overridable initializers)."""
        self._adapters.append(adapter)

    log_severity_level = property(lambda s: s._c.log_severity_level, lambda s, v: setattr(s._c, "log_severity_level", v))
    log_verbosity_level = property(lambda s: s._c.log_verbosity_level, lambda s, v: setattr(s._c, "log_verbosity_level", v))
    logid = property(lambda s: s._c.logid, lambda s, v: setattr(s._c, "logid", v))
    terminate = property(lambda s: s._c.terminate, lambda s, v: setattr(s._c, "terminate", bool(v)))
    only_execute_path_to_fetches = property(lambda s: s._c.only_execute_path_to_fetches,
                                            lambda s, v: setattr(s._c, "only_execute_path_to_fetches", bool(v)))

    def add_run_config_entry(self, key: str, value: str) -> None:
        self._c.add_config(key, str(value))

    def get_run_config_entry(self, key: str) -> str:
        v = self._c.get_config(key)
        if v is None:
            raise RuntimeException(f"Run config entry '{key}' was not found.")
        return v


# --------------------------------------------------------------- LoRA adapters
_ADAPTER_MAGIC = b"ORTB200ADAPTER\0\0"
_TORCH_TO_ONNX_ELEM = {torch.float32: 1, torch.uint8: 2, torch.int8: 3, torch.int16: 5, torch.int32: 6, torch.int64: 7,
                       torch.bool: 9, torch.float16: 10, torch.float64: 11, torch.bfloat16: 16,
                       torch.float8_e4m3fn: 17, torch.float8_e5m2: 19}


class AdapterFormat:
    """Adapter file: named parameters plus an adapter version and the version of the model they belong to
    (onnxruntime.AdapterFormat, onnxruntime/python/onnxruntime_inference_collection.py:67).  Files are written in the
    reference's own format - a FlatBuffer with file identifier ``TORT`` (``flatbuf_lite.py``) - so adapters travel in
    both directions; ``read_adapter`` also accepts the length-prefixed TensorProto container earlier versions of this
    package wrote (16-byte magic ``ORTB200ADAPTER``)."""

    def __init__(self):
        self._adapter_version = 1
        self._model_version = 1
        self._parameters: Dict[str, Any] = {}

    def set_adapter_version(self, v: int) -> None:
        self._adapter_version = int(v)

    def get_adapter_version(self) -> int:
        return self._adapter_version

    def set_model_version(self, v: int) -> None:
        self._model_version = int(v)

    def get_model_version(self) -> int:
        return self._model_version

    def set_parameters(self, params: Dict[str, Any]) -> None:
        self._parameters = dict(params)

    def get_parameters(self) -> Dict[str, "OrtValue"]:
        return {k: v if isinstance(v, OrtValue) else OrtValue(_to_torch(v)) for k, v in self._parameters.items()}

    def export_adapter(self, file_path: str) -> None:
        from . import flatbuf_lite as fb
        params = []
        for name, v in self._parameters.items():
            t = _to_torch(v).detach().cpu().contiguous()
            et = _TORCH_TO_ONNX_ELEM.get(t.dtype)
            if et is None:
                raise InvalidArgument(f"adapter parameter '{name}' has unsupported type {t.dtype}")
            raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
            params.append((name, list(t.shape), et, raw))
        with open(file_path, "wb") as f:
            f.write(fb.write_adapter(self._adapter_version, self._model_version, params))

    @staticmethod
    def read_adapter(file_path: str) -> "AdapterFormat":
        import struct
        from . import flatbuf_lite as fb
        with open(file_path, "rb") as f:
            buf = f.read()
        a = AdapterFormat()
        if fb.is_adapter_flatbuffer(buf):
            try:
                fmt, av, mv, params = fb.read_adapter(buf)
            except (ValueError, struct.error) as e:
                raise InvalidArgument(f"{file_path}: malformed adapter file ({e})") from None
            if fmt != fb.ADAPTER_FORMAT_VERSION:
                raise InvalidArgument(f"unsupported adapter format version {fmt}")
            a._adapter_version, a._model_version = av, mv
            onnx_to_torch = {v: k for k, v in _TORCH_TO_ONNX_ELEM.items()}
            for name, dims, et, raw in params:
                dt = onnx_to_torch.get(et)
                if dt is None:
                    raise InvalidArgument(f"adapter parameter '{name}' has unsupported element type {et}")
                t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dt) if raw else torch.empty(0, dtype=dt)
                a._parameters[name] = t.reshape(dims).clone()
            return a
        if buf[:16] != _ADAPTER_MAGIC:
            raise InvalidArgument(f"{file_path} is not an adapter file")
        fmt, av, mv, n = struct.unpack_from("<iiiI", buf, 16)
        if fmt != 1:
            raise InvalidArgument(f"unsupported adapter format version {fmt}")
        a._adapter_version, a._model_version = av, mv
        off = 32
        from . import onnx_lite as ol
        for _ in range(n):
            (ln,) = struct.unpack_from("<I", buf, off)
            off += 4
            blob = bytes(buf[off:off + ln])
            off += ln
            a._parameters[ol.load_tensor(blob).name] = C.tensor_from_proto(blob)
        return a


class LoraAdapter:
    """Adapter parameters kept ready for ``RunOptions.add_active_adapter`` (onnxruntime.LoraAdapter)."""

    def __init__(self):
        self._params: Dict[str, torch.Tensor] = {}

    def Load(self, file_path: str, device: Optional[str] = None) -> None:  # noqa: N802 (reference spelling)
        fmt = AdapterFormat.read_adapter(file_path)
        self._params = {k: (_to_torch(v).to(device) if device else _to_torch(v)) for k, v in fmt._parameters.items()}

    def parameters(self) -> Dict[str, torch.Tensor]:
        return self._params


def register_custom_op(domain: str, op_type: str, fn) -> None:
    """Register a Python callable as the kernel of ``domain::op_type``.

    ``fn(*inputs, **attributes)`` receives torch tensors (``None`` for omitted optional inputs; on the device the
    node runs on) and the node's attributes, and returns one tensor or a tuple of tensors.  The registration is
    process-wide and must happen before the sessions that use the operator are created."""
    C.register_python_op(domain, op_type, fn)


def _image_decoder(encoded_stream, pixel_format="RGB", **_unused):
    """ONNX ImageDecoder (opset 20): encoded image bytes (JPEG, PNG, BMP, ...) -> [H, W, C] uint8 in RGB, BGR or Grayscale.
    Decoding is Pillow's, so this operator runs as a Python callable registered with the kernel registry when the package
    is imported (the registry has no image codec of its own)."""
    import io

    from PIL import Image
    fmt = pixel_format.decode() if isinstance(pixel_format, bytes) else str(pixel_format)
    img = Image.open(io.BytesIO(bytes(encoded_stream.cpu().numpy().astype(np.uint8).tobytes())))
    if fmt == "Grayscale":
        arr = np.asarray(img.convert("L"))[:, :, None]
    else:
        arr = np.asarray(img.convert("RGB"))
        if fmt == "BGR":
            arr = arr[:, :, ::-1]
        elif fmt != "RGB":
            raise InvalidArgument(f"ImageDecoder: unknown pixel_format '{fmt}'")
    return torch.from_numpy(np.array(arr, copy=True))


try:
    C.register_python_op("", "ImageDecoder", _image_decoder)
except Exception:  # pragma: no cover - the native module decides whether Python operators are available
    pass


# --------------------------------------------------------------- provider args
def check_and_normalize_provider_args(providers, provider_options, available) -> Tuple[List[str], List[Dict[str, str]]]:
    """Same contract as the reference helper (onnxruntime_inference_collection.py:119)."""
    if providers is None:
        return [], []
    if not isinstance(providers, Sequence) or isinstance(providers, str):
        raise ValueError("'providers' should be a sequence.")
    names: List[str] = []
    opts: List[Dict[str, str]] = []

    def add(name, options):
        if name not in _ALL_PROVIDERS:
            raise ValueError(f"Specified provider '{name}' is not in available provider names."
                             f"Available providers: '{', '.join(available)}'")
        if name in names:
            return
        names.append(name)
        opts.append({str(k): str(v) for k, v in (options or {}).items()})

    if provider_options is not None:
        if not isinstance(provider_options, Sequence) or len(provider_options) != len(providers):
            raise ValueError("'provider_options' should be a sequence with the same length as 'providers'.")
        for p, o in zip(providers, provider_options):
            if not isinstance(p, str) or not isinstance(o, dict):
                raise ValueError("'providers' values must be strings and 'provider_options' values must be dicts")
            add(p, o)
    else:
        for p in providers:
            if isinstance(p, str):
                add(p, {})
            elif isinstance(p, tuple) and len(p) == 2 and isinstance(p[0], str) and isinstance(p[1], dict):
                add(p[0], p[1])
            else:
                raise ValueError("'providers' values must be either provider names or (name, options dict) tuples.")
    return names, opts


# ------------------------------------------------------------- InferenceSession
class InferenceSession:
    """Load an ONNX model and run it.

    ``InferenceSession(path_or_bytes, sess_options=None, providers=None, provider_options=None)``;
    keyword extras: ``disabled_optimizers`` (list of pass names), ``enable_fallback``.
    """

    def __init__(self, path_or_bytes: Union[str, bytes, os.PathLike], sess_options: Optional[SessionOptions] = None,
                 providers=None, provider_options=None, **kwargs):
        self._sess_options = sess_options if sess_options is not None else SessionOptions()
        self._enable_fallback = bool(kwargs.get("enable_fallback", True))
        disabled = list(kwargs.get("disabled_optimizers") or [])
        if isinstance(path_or_bytes, (str, os.PathLike)):
            self._model_path = os.fspath(path_or_bytes)
            self._model_bytes = None
        elif isinstance(path_or_bytes, (bytes, bytearray, memoryview)):
            self._model_path = None
            self._model_bytes = bytes(path_or_bytes)
        else:
            raise TypeError(f"Unable to load from type '{type(path_or_bytes)}'")
        available = get_available_providers()
        so = self._sess_options
        if getattr(so, "_load_cancelled", False):
            raise ModelLoadCanceled("the session options' load cancellation flag is set")
        if providers is None and getattr(so, "_providers_for_devices", None):
            providers = [n for n, _ in so._providers_for_devices]
            provider_options = [o for _, o in so._providers_for_devices]
        if providers is None and getattr(so, "_selection_delegate", None) is not None:
            picked = so._selection_delegate(get_ep_devices(), {}, {}, 8)
            providers = list(dict.fromkeys(d.ep_name for d in picked))
        if providers is None and getattr(so, "_selection_policy", OrtExecutionProviderDevicePolicy.DEFAULT) != OrtExecutionProviderDevicePolicy.DEFAULT:
            gpu = so._selection_policy in (OrtExecutionProviderDevicePolicy.PREFER_GPU, OrtExecutionProviderDevicePolicy.MAX_PERFORMANCE)
            providers = ["CUDAExecutionProvider", "CPUExecutionProvider"] if gpu and torch.cuda.is_available() else ["CPUExecutionProvider"]
        names, opts = check_and_normalize_provider_args(providers, provider_options, available)
        if not names:
            names, opts = ["CPUExecutionProvider"], [{}]
        self._fallback_providers = ["CPUExecutionProvider"]
        self._dist = kwargs.get("dist")
        try:
            self._create(names, opts, disabled)
        except (EPFail, RuntimeException) as e:
            if not self._enable_fallback or names == self._fallback_providers:
                raise
            import warnings
            warnings.warn(f"EP Error {e} when using {names}; falling back to {self._fallback_providers} and retrying.")
            self._create(self._fallback_providers, [{}], disabled)
        self._lock = threading.Lock()

    def _create(self, names, opts, disabled) -> None:
        if "CUDAExecutionProvider" in names and not torch.cuda.is_available():
            if names == ["CUDAExecutionProvider"] and not self._enable_fallback:
                raise EPFail("CUDAExecutionProvider requested but no CUDA device is available")
            pairs = [(n, o) for n, o in zip(names, opts) if n != "CUDAExecutionProvider"]
            names, opts = [p[0] for p in pairs] or ["CPUExecutionProvider"], [p[1] for p in pairs] or [{}]
        sess = C.InferenceSession(self._sess_options._c)
        cfg = self._sess_options._c.config_entries()
        load_format = cfg.get("session.load_model_format", "").upper()
        if self._model_path is not None and (load_format == "ORT" or (load_format == "" and self._model_path.lower().endswith(".ort"))):
            with open(self._model_path, "rb") as f:
                self._model_bytes, self._model_path = f.read(), None
        if self._model_bytes is not None and (load_format == "ORT" or (load_format == "" and _is_ort_format(self._model_bytes))):
            # ORT-format (FlatBuffers) model: converted to the ONNX form the core loads (ort_format.py)
            from . import ort_format
            try:
                self._model_bytes = ort_format.ort_to_onnx(self._model_bytes).serialize()
            except (ValueError, struct_error) as e:
                raise InvalidProtobuf(f"cannot read the ORT-format model: {e}") from None
        ext_files = getattr(self._sess_options, "_external_files", None)
        if ext_files:
            # external-data files handed over as memory: put their bytes into the initializers that point to them
            from . import onnx_lite as ol
            model = ol.load_model(self._model_path if self._model_path is not None else self._model_bytes)

            def inline(graph):
                for t in graph.initializers:
                    loc = (t.external or {}).get("location")
                    if loc is None or loc == "*session*":
                        continue
                    data = ext_files.get(loc, ext_files.get(os.path.basename(loc)))
                    if data is None:
                        continue
                    off = int(t.external.get("offset", 0))
                    ln = int(t.external["length"]) if "length" in t.external else len(data) - off
                    if off + ln > len(data):
                        raise InvalidArgument(f"initializer '{t.name}' reads bytes [{off}, {off + ln}) of '{loc}', which holds {len(data)}")
                    t.raw, t.external = data[off:off + ln], None
                for node in graph.nodes:
                    for a in node.attributes:
                        if a.type == ol.ATTR_GRAPH:
                            inline(a.value)
            inline(model.graph)
            model_dir = os.path.dirname(self._model_path) if self._model_path is not None else None
            self._model_bytes = model.serialize()
            if model_dir and any((t.external or {}).get("location") not in (None, "*session*") for t in model.graph.initializers):
                # some initializers still live in real files next to the model: keep loading from that directory
                tmp = os.path.join(model_dir, f".ortb200_inline_{os.getpid()}.onnx")
                with open(tmp, "wb") as f:
                    f.write(self._model_bytes)
                try:
                    sess.load(tmp)
                finally:
                    os.remove(tmp)
            else:
                sess.load_bytes(self._model_bytes)
        elif self._model_path is not None:
            sess.load(self._model_path)
        else:
            sess.load_bytes(self._model_bytes)
        dist = self._dist
        if dist is not None:
            sess.dist_group = dist.group_name
            sess.rank = dist.rank
            sess.world_size = dist.world_size
        sess.initialize(list(zip(names, opts)), disabled)
        self._sess = sess
        out_path = self._sess_options.optimized_model_filepath
        save_format = cfg.get("session.save_model_format", "").upper()
        if out_path and (save_format == "ORT" or (save_format == "" and out_path.lower().endswith(".ort"))):
            # the core wrote the optimized model as ONNX; rewrite it in the ORT format
            from . import onnx_lite as ol, ort_format
            with open(out_path, "rb") as f:
                optimized = ol.load_model(f.read())
            with open(out_path, "wb") as f:
                f.write(ort_format.onnx_to_ort(optimized))
        self._providers = sess.providers()
        self._provider_options = sess.provider_options()
        self._inputs_meta = [NodeArg(m) for m in sess.inputs_meta()]
        self._outputs_meta = [NodeArg(m) for m in sess.outputs_meta()]
        self._overridable = [NodeArg(m) for m in sess.overridable_initializers_meta()]
        self._input_names = [m.name for m in self._inputs_meta]

    # --- metadata
    def get_session_options(self) -> SessionOptions:
        return self._sess_options

    def get_inputs(self) -> List[NodeArg]:
        return self._inputs_meta

    def get_outputs(self) -> List[NodeArg]:
        return self._outputs_meta

    def get_overridable_initializers(self) -> List[NodeArg]:
        return self._overridable

    def get_modelmeta(self) -> ModelMetadata:
        return ModelMetadata(self._sess.model_meta())

    def get_providers(self) -> List[str]:
        return list(self._providers)

    def get_provider_options(self) -> Dict[str, Dict[str, str]]:
        return {k: dict(v) for k, v in self._provider_options.items()}

    def set_providers(self, providers=None, provider_options=None) -> None:
        names, opts = check_and_normalize_provider_args(providers, provider_options, get_available_providers())
        self._create(names or ["CPUExecutionProvider"], opts or [{}], [])

    def get_provider_graph_assignment_info(self):
        return self._sess.node_assignments()

    def get_profiling_start_time_ns(self) -> int:
        return self._sess.profiling_start_time_ns()

    def end_profiling(self) -> str:
        return self._sess.end_profiling()

    # --- running
    def _validate_input(self, feed_names: Sequence[str]) -> None:
        missing = [n for n in self._input_names if n not in feed_names]
        if missing:
            raise ValueError(f"Required inputs ({missing}) are missing from input feed ({list(feed_names)}).")

    def run(self, output_names: Optional[Sequence[str]], input_feed: Dict[str, Any],
            run_options: Optional[RunOptions] = None) -> List[Any]:
        self._validate_input(list(input_feed.keys()))
        ro = run_options._c if run_options is not None else C.RunOptions()
        input_feed = self._with_adapters(input_feed, run_options)
        names = list(input_feed.keys())
        feeds = [_to_torch(v) for v in input_feed.values()]
        outs = self._sess.run(ro, names, feeds, list(output_names or []))
        return [_to_numpy(o) for o in outs]

    def _with_adapters(self, input_feed: Dict[str, Any], run_options: Optional[RunOptions]) -> Dict[str, Any]:
        if run_options is None or not run_options._adapters:
            return input_feed
        accepted = {a.name for a in self.get_inputs()} | {a.name for a in self.get_overridable_initializers()}
        merged = dict(input_feed)
        for adapter in run_options._adapters:
            for name, value in adapter.parameters().items():
                if name in accepted and name not in input_feed:
                    merged[name] = value
        return merged

    def run_with_ort_values(self, output_names: Optional[Sequence[str]], input_dict_ort_values: Dict[str, OrtValue],
                            run_options: Optional[RunOptions] = None) -> List[OrtValue]:
        self._validate_input(list(input_dict_ort_values.keys()))
        ro = run_options._c if run_options is not None else C.RunOptions()
        input_dict_ort_values = self._with_adapters(input_dict_ort_values, run_options)
        names = list(input_dict_ort_values.keys())
        feeds = [_to_torch(v) for v in input_dict_ort_values.values()]
        outs = self._sess.run(ro, names, feeds, list(output_names or []))
        # a string output comes back as ("__strings__", values, shape)
        return [OrtValue(_StringTensor(o[1], o[2]) if isinstance(o, tuple) and len(o) == 3 and o[0] == "__strings__" else o) for o in outs]

    def run_with_ortvaluevector(self, run_options, feed_names: Sequence[str], feeds: "OrtValueVector", fetch_names: Sequence[str],
                                fetches: "OrtValueVector", fetch_devices: Sequence[OrtDevice]) -> None:
        """Run with OrtValue vectors: `fetches` is filled with one OrtValue per fetch name, placed on `fetch_devices`."""
        if len(feed_names) != len(feeds):
            raise InvalidArgument("feed_names and feeds differ in length")
        if len(fetch_devices) != len(fetch_names):
            raise InvalidArgument("fetch_names and fetch_devices differ in length")
        ro = run_options._c if run_options is not None else C.RunOptions()
        outs = self._sess.run(ro, list(feed_names), [_to_torch(v) for v in feeds], list(fetch_names))
        fetches.clear()
        for o, dev in zip(outs, fetch_devices):
            if isinstance(o, torch.Tensor):
                o = o.to(dev._torch() if isinstance(dev, OrtDevice) else torch.device(dev))
            fetches.push_back(OrtValue(o))

    def run_async(self, output_names, input_feed, callback, user_data, run_options=None) -> None:
        def work():
            try:
                res = self.run(output_names, input_feed, run_options)
                callback(res, user_data, "")
            except Exception as e:  # the callback receives the error text, as in the reference
                callback(None, user_data, str(e))
        threading.Thread(target=work, daemon=True).start()

    def io_binding(self) -> "IOBinding":
        return IOBinding(self)

    def run_with_iobinding(self, iobinding: "IOBinding", run_options: Optional[RunOptions] = None) -> None:
        ro = run_options._c if run_options is not None else C.RunOptions()
        if iobinding._has_strings():
            iobinding._run_by_name(ro)
            return
        iobinding._string_results = None
        self._sess.run_with_binding(ro, iobinding._c)

    # --- extras of this runtime
    def graph_nodes(self) -> List[Dict[str, Any]]:
        """The optimized, partitioned graph as a list of node dicts (op_type, domain, inputs, outputs, ep, attrs)."""
        return self._sess.graph_nodes()

    def serialize_optimized_model(self) -> bytes:
        return self._sess.serialize_model()

    def kernel_launch_count(self) -> int:
        return self._sess.kernel_launch_count()

    def last_run_launch_count(self) -> int:
        """Kernels of this library launched by the most recent eager run (or captured into the most recent graph)."""
        return self._sess.last_run_launch_count()

    def num_captured_graphs(self) -> int:
        return self._sess.num_captured_graphs()

    def check_device_status(self) -> None:
        self._sess.check_device_status()

    def get_memory_plans(self):
        """One entry per input-shape pattern run so far (``SessionOptions.enable_mem_pattern``): the arena size that
        would serve the pattern with buffer reuse (``*_peak_bytes``), the sum of all requests (``*_total_bytes``), the
        lower bound (``*_live_peak_bytes``) and per value ``(name, bytes, first_step, last_step, on_gpu, offset)``.
        The reference keeps the same information in its memory-pattern planner
        (onnxruntime/core/framework/mem_pattern_planner.h)."""
        return self._sess.memory_plans()

    _TUNING_VALIDATORS = {"ORTB200_VERSION": "0.1.0", "DEVICE_ARCH": "sm_100a"}

    def get_tuning_results(self) -> List[dict]:
        """TunableOp results in the reference's shape (``InferenceSession.get_tuning_results``): one entry per
        provider with ``results[op][signature] = configuration`` and the validators that must match on import."""
        res = self._sess.tuning_results()
        if not res:
            return []
        gemm = {k: f"splits={v[0]},bn={v[1]},tile_rows={v[2]}" for k, v in res.items()}
        return [{"ep": "CUDAExecutionProvider", "results": {"Gemm": gemm}, "validators": dict(self._TUNING_VALIDATORS)}]

    def set_tuning_results(self, results: List[dict], *, error_on_invalid: bool = False) -> None:
        for entry in results or []:
            ok = entry.get("ep") == "CUDAExecutionProvider" and entry.get("validators") == self._TUNING_VALIDATORS
            if not ok:
                if error_on_invalid:
                    raise InvalidArgument("tuning results were recorded by another provider, version or device architecture")
                continue
            for sig, cfg in entry.get("results", {}).get("Gemm", {}).items():
                try:
                    kv = dict(item.split("=") for item in cfg.split(","))
                    self._sess.set_tuning_result(sig, int(kv["splits"]), int(kv["bn"]), int(kv["tile_rows"]))
                except (KeyError, ValueError):
                    if error_on_invalid:
                        raise InvalidArgument(f"malformed tuning result for {sig}: {cfg!r}") from None

    def get_memory_stats(self) -> dict:
        """Statistics of the device arena (the torch caching allocator) for a GPU session; empty for CPU sessions."""
        return self._sess.memory_stats()


# --------------------------------------------------------------------- compile API
class ModelCompiler:
    """Ahead-of-time preparation of a model: the graph is optimized, fused and lowered for the providers given in the
    session options, and stored as a model with one ``com.microsoft.EPContext`` node whose payload is that graph; a
    session created from the result skips the preparation.  Mirrors the reference's ``onnxruntime.ModelCompiler``
    (onnxruntime/python/onnxruntime_inference_collection.py; C side onnxruntime/core/session/compile_api.cc) and the
    ``ep.context_*`` session configuration keys.

    ``input_model`` is a path or the model's bytes.  ``embed_compiled_data_into_model`` = False puts the payload
    into a side file beside the output model (``compile_to_file`` only)."""

    def __init__(self, sess_options: Optional["SessionOptions"], input_model, embed_compiled_data_into_model: bool = False,
                 providers=None, provider_options=None, **kwargs):
        self._so = sess_options
        self._input = input_model
        self._embed = bool(embed_compiled_data_into_model)
        self._providers = providers
        self._provider_options = provider_options
        self._kwargs = kwargs

    def _options(self, out_path: str, embed: bool) -> "SessionOptions":
        so = SessionOptions()
        if self._so is not None:
            for f in SessionOptions._FIELDS:
                setattr(so, f, getattr(self._so, f))
            so.graph_optimization_level = self._so.graph_optimization_level
            so.execution_mode = self._so.execution_mode
            for k, v in self._so._c.config_entries().items():
                so.add_session_config_entry(k, v)
        so.add_session_config_entry("ep.context_enable", "1")
        so.add_session_config_entry("ep.context_file_path", out_path)
        so.add_session_config_entry("ep.context_embed_mode", "1" if embed else "0")
        return so

    def compile_to_file(self, output_model_path: str) -> None:
        InferenceSession(self._input, self._options(os.fspath(output_model_path), self._embed), providers=self._providers,
                         provider_options=self._provider_options, **self._kwargs)

    def compile_to_bytes(self) -> bytes:
        import tempfile
        with tempfile.TemporaryDirectory() as d:
            out = os.path.join(d, "compiled.onnx")
            InferenceSession(self._input, self._options(out, True), providers=self._providers,
                             provider_options=self._provider_options, **self._kwargs)
            with open(out, "rb") as f:
                return f.read()


# --------------------------------------------------------------------- IOBinding
class IOBinding:
    """Bind model inputs/outputs to caller-owned (possibly device) buffers."""

    def __init__(self, session: InferenceSession):
        self._session = session
        self._c = C.IOBinding(session._sess)
        self._keep: List[Any] = []
        # Tensors of strings have no device buffer to bind: a binding that holds one runs through the by-name path,
        # with every bound input kept here by name and bound output buffers filled by copy.
        self._inputs: Dict[str, Any] = {}
        self._out_buffers: Dict[str, Optional[torch.Tensor]] = {}
        self._string_results: Optional[List[Any]] = None
        self._string_outputs: Optional[bool] = None
        self._string_inputs = 0

    def _has_strings(self) -> bool:   # on the path of every bound run: two attribute reads
        if self._string_outputs is None:
            self._string_outputs = any(o.type == "tensor(string)" for o in self._session.get_outputs())
        return self._string_outputs or self._string_inputs > 0

    def _run_by_name(self, run_options) -> None:
        wanted = list(self._out_buffers) or [o.name for o in self._session.get_outputs()]
        outs = self._session._sess.run(run_options, list(self._inputs), list(self._inputs.values()), wanted)
        for name, value in zip(wanted, outs):
            buf = self._out_buffers.get(name)
            if buf is not None and isinstance(value, torch.Tensor):
                buf.copy_(value)
        self._string_results = [_StringTensor(o[1], o[2]) if isinstance(o, tuple) and len(o) == 3 and o[0] == "__strings__" else o
                                for o in outs]

    def bind_cpu_input(self, name: str, arr_on_cpu: np.ndarray) -> None:
        t = _to_torch(arr_on_cpu)
        self._inputs[name] = t
        if isinstance(t, _StringTensor):
            self._string_inputs += 1
        else:
            self._c.bind_input(name, t)

    def bind_input(self, name: str, device_type: str, device_id: int, element_type, shape: Sequence[int],
                   buffer_ptr: int) -> None:
        t = _tensor_from_pointer(buffer_ptr, element_type, shape, device_type, device_id)
        self._keep.append(t)
        self._inputs[name] = t
        self._c.bind_input(name, t)

    def bind_ortvalue_input(self, name: str, ortvalue: OrtValue) -> None:
        t = _to_torch(ortvalue)
        self._inputs[name] = t
        if isinstance(t, _StringTensor):
            self._string_inputs += 1
        else:
            self._c.bind_input(name, t)

    def bind_torch_input(self, name: str, tensor: torch.Tensor) -> None:
        self._inputs[name] = tensor
        self._c.bind_input(name, tensor)

    def bind_output(self, name: str, device_type: str = "cpu", device_id: int = 0, element_type=None,
                    shape: Optional[Sequence[int]] = None, buffer_ptr: Optional[int] = None) -> None:
        if buffer_ptr is None:
            self._out_buffers[name] = None
            self._c.bind_output_to_device(name, device_type.lower(), device_id)
            return
        if element_type is None or shape is None:
            raise InvalidArgument("`element_type` and `shape` are to be provided if pre-allocated memory is provided")
        t = _tensor_from_pointer(buffer_ptr, element_type, shape, device_type, device_id)
        self._keep.append(t)
        self._out_buffers[name] = t
        self._c.bind_output(name, t)

    def bind_ortvalue_output(self, name: str, ortvalue: OrtValue) -> None:
        self._out_buffers[name] = _to_torch(ortvalue)
        self._c.bind_output(name, self._out_buffers[name])

    def bind_torch_output(self, name: str, tensor: torch.Tensor) -> None:
        self._out_buffers[name] = tensor
        self._c.bind_output(name, tensor)

    def synchronize_inputs(self) -> None:
        self._c.synchronize_inputs()

    def synchronize_outputs(self) -> None:
        self._c.synchronize_outputs()

    def get_outputs(self) -> List[OrtValue]:
        if self._string_results is not None:
            return [OrtValue(t) for t in self._string_results]
        return [OrtValue(t) for t in self._c.results()]

    def copy_outputs_to_cpu(self) -> List[np.ndarray]:
        if self._string_results is not None:
            return [t.numpy() if isinstance(t, _StringTensor) else _to_numpy(t) for t in self._string_results]
        return [_to_numpy(t) for t in self._c.results()]

    def clear_binding_inputs(self) -> None:
        self._inputs.clear()
        self._string_inputs = 0
        self._c.clear_inputs()

    def clear_binding_outputs(self) -> None:
        self._out_buffers.clear()
        self._string_results = None
        self._c.clear_outputs()
        self._keep.clear()


def _tensor_from_pointer(ptr: int, element_type, shape, device_type: str, device_id: int) -> torch.Tensor:
    """Wrap foreign memory (no copy) as a torch tensor."""
    if isinstance(element_type, int):
        dt = _ONNX_ELEM_TO_TORCH[element_type]
    elif isinstance(element_type, torch.dtype):
        dt = element_type
    else:
        dt = torch.from_numpy(np.zeros((), dtype=element_type)).dtype
    numel = int(np.prod(shape)) if len(shape) else 1
    nbytes = numel * torch.empty((), dtype=dt).element_size()
    if device_type.lower() == "cuda":
        class _Holder:
            pass
        h = _Holder()
        h.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}
        raw = torch.as_tensor(h, device=torch.device("cuda", device_id))
    else:
        import ctypes
        buf = (ctypes.c_uint8 * nbytes).from_address(int(ptr))
        raw = torch.frombuffer(buf, dtype=torch.uint8)
    return raw.view(dt).reshape(tuple(shape))
