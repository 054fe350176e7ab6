"""On-device training API: ``CheckpointState``, ``Module``, ``Optimizer``, ``LinearLRScheduler``.

Same surface as the reference's ``onnxruntime.training.api`` (``orttraining/orttraining/python/training/api/``,
implemented natively in ``orttraining/orttraining/training_api/{module,optimizer,checkpoint,lr_scheduler}.cc``), over
the artifacts of ``generate_artifacts``.  Parameters, gradient buffers and optimizer moments are torch tensors that the
training and optimizer graphs update in place (``InPlaceAccumulatorV2``, ``AdamWOptimizer``), on the CPU or on a GPU.

The checkpoint is one file: a little-endian header ``b"ORTB200CKPT"``, a JSON index (names, dtypes, shapes, offsets,
trainable flags, properties, optimizer step) and the raw tensor bytes, each 64-byte aligned so that a reader can map it.
"""
from __future__ import annotations

import io
import json
import struct
from typing import Dict, Iterable, List, Optional, Sequence, Set, Union

import numpy as np
import torch

_MAGIC = b"ORTB200CKPT"


def _np(t) -> np.ndarray:
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu()
        return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()
    return np.asarray(t)


class Parameter:
    """One named parameter: its value, whether it is trained, and its gradient buffer."""

    def __init__(self, name: str, data: torch.Tensor, requires_grad: bool):
        self.name, self.data, self.requires_grad = name, data, requires_grad
        self.grad: Optional[torch.Tensor] = torch.zeros_like(data) if requires_grad else None


class CheckpointState:
    def __init__(self):
        self.parameters: Dict[str, Parameter] = {}
        self.optimizer: Dict[str, Dict[str, torch.Tensor]] = {}    # "momentum0" / "momentum1" -> name -> tensor
        self.optimizer_step: int = 0
        self.learning_rate: Optional[float] = None
        self.properties: Dict[str, Union[int, float, str]] = {}

    @classmethod
    def from_parameters(cls, values: Dict[str, np.ndarray], trainable: Set[str]) -> "CheckpointState":
        s = cls()
        for name, arr in values.items():
            s.parameters[name] = Parameter(name, torch.from_numpy(np.array(arr)), name in trainable)
        return s

    # ---- serialisation
    def to_bytes(self) -> bytes:
        index = {"parameters": [], "optimizer": [], "step": self.optimizer_step, "lr": self.learning_rate, "properties": self.properties}
        blobs: List[bytes] = []
        offset = 0

        def put(t: torch.Tensor) -> Dict[str, object]:
            nonlocal offset
            raw = _np(t.contiguous()).tobytes()
            pad = (-len(raw)) % 64
            entry = {"dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape), "offset": offset, "nbytes": len(raw)}
            blobs.append(raw + b"\0" * pad)
            offset += len(raw) + pad
            return entry
        for p in self.parameters.values():
            index["parameters"].append({"name": p.name, "requires_grad": p.requires_grad, **put(p.data)})
        for group, tensors in self.optimizer.items():
            for name, t in tensors.items():
                index["optimizer"].append({"group": group, "name": name, **put(t)})
        head = json.dumps(index).encode()
        head += b" " * ((-(len(_MAGIC) + 8 + len(head))) % 64)
        return _MAGIC + struct.pack("<Q", len(head)) + head + b"".join(blobs)

    @classmethod
    def from_bytes(cls, blob: bytes) -> "CheckpointState":
        if blob[:len(_MAGIC)] != _MAGIC:
            raise ValueError("not a checkpoint of this runtime")
        (n,) = struct.unpack_from("<Q", blob, len(_MAGIC))
        start = len(_MAGIC) + 8
        index = json.loads(blob[start:start + n].decode())
        base = start + n

        def get(e) -> torch.Tensor:
            dt = getattr(torch, e["dtype"])
            raw = bytearray(blob[base + e["offset"]: base + e["offset"] + e["nbytes"]])
            return torch.frombuffer(raw, dtype=dt).reshape(e["shape"]).clone() if e["nbytes"] else torch.zeros(e["shape"], dtype=dt)
        s = cls()
        for e in index["parameters"]:
            s.parameters[e["name"]] = Parameter(e["name"], get(e), bool(e["requires_grad"]))
        for e in index["optimizer"]:
            s.optimizer.setdefault(e["group"], {})[e["name"]] = get(e)
        s.optimizer_step, s.learning_rate, s.properties = int(index["step"]), index["lr"], dict(index["properties"])
        return s

    @staticmethod
    def load_checkpoint(path_or_bytes: Union[str, bytes]) -> "CheckpointState":
        if isinstance(path_or_bytes, (bytes, bytearray)):
            return CheckpointState.from_bytes(bytes(path_or_bytes))
        with open(path_or_bytes, "rb") as f:
            return CheckpointState.from_bytes(f.read())

    @staticmethod
    def save_checkpoint(state: "CheckpointState", path: str, include_optimizer_state: bool = True) -> None:
        saved = state.optimizer
        if not include_optimizer_state:
            state.optimizer = {}
        try:
            with open(path, "wb") as f:
                f.write(state.to_bytes())
        finally:
            state.optimizer = saved


class Module:
    """Runs the training model (loss + gradient accumulation) or the eval model over the parameters of a checkpoint."""

    def __init__(self, train_model: Union[str, bytes], state: CheckpointState, eval_model: Optional[Union[str, bytes]] = None,
                 device: str = "cpu"):
        from .. import capi
        self._C = capi.C
        self._state = state
        self._device = torch.device(device)
        providers = ["CPUExecutionProvider"] if self._device.type == "cpu" else [("CUDAExecutionProvider", {"device_id": self._device.index or 0}), "CPUExecutionProvider"]
        so = capi.SessionOptions()
        so.graph_optimization_level = capi.GraphOptimizationLevel.ORT_ENABLE_BASIC
        if self._device.type != "cpu":
            so.add_session_config_entry("ortb200.generic_kernels_only", "1")   # the hand-written kernels are inference-only
        self._eval_source = eval_model
        self._train = capi.InferenceSession(train_model, so, providers=providers)
        self._eval = capi.InferenceSession(eval_model, so, providers=providers) if eval_model is not None else None
        for p in state.parameters.values():
            p.data = p.data.to(self._device)
            if p.grad is not None:
                p.grad = p.grad.to(self._device)
        self._training = True
        self._reset = True
        names = set(state.parameters)
        skip = names | {n + "_grad.accumulation.buffer" for n in names} | {"lazy_reset_grad"}
        self._train_inputs = [i.name for i in self._train.get_inputs() if i.name not in skip]
        self._train_outputs = [o.name for o in self._train.get_outputs() if not o.name.endswith("_grad.accumulation.out")]
        self._flag_outputs = [o.name for o in self._train.get_outputs() if o.name.endswith("_grad.accumulation.out")]
        if self._eval is not None:
            self._eval_inputs = [i.name for i in self._eval.get_inputs() if i.name not in names]
            self._eval_outputs = [o.name for o in self._eval.get_outputs()]

    def train(self, mode: bool = True) -> None:
        self._training = mode

    def eval(self) -> None:
        self._training = False

    def lazy_reset_grad(self) -> None:
        """The next training step overwrites the gradient buffers instead of adding to them."""
        self._reset = True

    def input_names(self) -> List[str]:
        return list(self._train_inputs if self._training or self._eval is None else self._eval_inputs)

    def output_names(self) -> List[str]:
        return list(self._train_outputs if self._training or self._eval is None else self._eval_outputs)

    def parameters(self) -> List[Parameter]:
        return list(self._state.parameters.values())

    def named_parameters(self):
        return list(self._state.parameters.items())

    def get_parameters_size(self, trainable_only: bool = True) -> int:
        return sum(p.data.numel() for p in self.parameters() if p.requires_grad or not trainable_only)

    def get_contiguous_parameters(self, trainable_only: bool = False) -> torch.Tensor:
        return torch.cat([p.data.reshape(-1).to(torch.float32) for p in self.parameters() if p.requires_grad or not trainable_only])

    def copy_buffer_to_parameters(self, buffer: torch.Tensor, trainable_only: bool = True) -> None:
        at = 0
        for p in self.parameters():
            if p.requires_grad or not trainable_only:
                n = p.data.numel()
                p.data.copy_(buffer[at:at + n].reshape(p.data.shape).to(p.data.dtype))
                at += n

    def all_reduce_gradients(self, group=None, average: bool = True, bucket_bytes: int = 256 << 20) -> None:
        """Data parallelism: sums (or averages) the gradient buffers over the ranks of ``group`` (``torch.distributed``;
        NCCL over NVLink for GPU modules, gloo on the CPU).  Gradients of one dtype travel as flat buckets of up to
        ``bucket_bytes``, so the cost is a few collective launches rather than one per parameter (the role of the
        reference's ``NcclAllReduce`` nodes that its data-parallel graph transform adds)."""
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
            return
        world = dist.get_world_size(group)
        pending: List[torch.Tensor] = []
        size = 0

        def flush() -> None:
            nonlocal pending, size
            if not pending:
                return
            flat = torch.cat([g.reshape(-1) for g in pending])
            dist.all_reduce(flat, group=group)
            if average:
                flat.div_(world)
            at = 0
            for g in pending:
                g.copy_(flat[at:at + g.numel()].reshape(g.shape))
                at += g.numel()
            pending, size = [], 0
        by_dtype: Dict[torch.dtype, List[torch.Tensor]] = {}
        for p in self.parameters():
            if p.requires_grad:
                by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
        for grads in by_dtype.values():
            for g in grads:
                if size and size + g.numel() * g.element_size() > bucket_bytes:
                    flush()
                pending.append(g)
                size += g.numel() * g.element_size()
            flush()

    def _tensor(self, v) -> torch.Tensor:
        t = v if isinstance(v, torch.Tensor) else torch.as_tensor(np.asarray(v))
        return t.to(self._device)

    def __call__(self, *inputs):
        training = self._training or self._eval is None
        sess = self._train if training else self._eval
        in_names = self._train_inputs if training else self._eval_inputs
        if len(inputs) != len(in_names):
            raise ValueError(f"expected inputs {in_names}, got {len(inputs)} values")
        names = list(in_names)
        values = [self._tensor(v) for v in inputs]
        for p in self._state.parameters.values():
            names.append(p.name)
            values.append(p.data)
            if training and p.requires_grad:
                names.append(p.name + "_grad.accumulation.buffer")
                values.append(p.grad)
        wanted = list(self._train_outputs if training else self._eval_outputs)
        if training:
            names.append("lazy_reset_grad")
            values.append(torch.tensor([self._reset]))
            wanted += self._flag_outputs
        with torch.no_grad():
            outs = sess._sess.run(self._C.RunOptions(), names, values, wanted)
        if training:
            self._reset = False
            outs = outs[:len(self._train_outputs)]
        outs = [o.detach().cpu().numpy() if isinstance(o, torch.Tensor) else o for o in outs]
        return outs[0] if len(outs) == 1 else tuple(outs)

    def export_model_for_inferencing(self, path: str, graph_output_names: Sequence[str]) -> None:
        """Writes the eval graph with the present parameter values as initializers and only the named outputs."""
        from .. import onnx_lite as ol
        if self._eval is None:
            raise RuntimeError("an eval model is needed to export for inferencing")
        m = ol.load_model(self._eval_source)
        g = m.graph
        names = set(self._state.parameters)
        g.inputs[:] = [v for v in g.inputs if v.name not in names]
        for p in self._state.parameters.values():
            g.initializers.append(ol.make_tensor(p.name, p.data.detach().cpu()))
        keep = set(graph_output_names)
        all_outs = {o.name: o for o in g.outputs}
        g.outputs[:] = [all_outs.get(n) or ol.make_tensor_value_info(n, 0, None) for n in graph_output_names]
        needed, nodes = set(keep), []
        for n in reversed(g.nodes):
            if any(o in needed for o in n.outputs):
                nodes.append(n)
                needed.update(i for i in n.inputs if i)
        g.nodes[:] = list(reversed(nodes))
        g.inputs[:] = [v for v in g.inputs if v.name in needed]
        with open(path, "wb") as f:
            f.write(m.serialize())


class Optimizer:
    def __init__(self, optimizer_model: Union[str, bytes], module: Module):
        from .. import capi, onnx_lite as ol
        self._C = capi.C
        self._module = module
        m = ol.load_model(optimizer_model)
        self._kind = m.metadata.get("optimizer", "AdamW")
        so = capi.SessionOptions()
        so.graph_optimization_level = capi.GraphOptimizationLevel.ORT_DISABLE_ALL
        providers = ["CPUExecutionProvider"] if module._device.type == "cpu" else [("CUDAExecutionProvider", {"device_id": module._device.index or 0}), "CPUExecutionProvider"]
        self._sess = capi.InferenceSession(optimizer_model, so, providers=providers)
        state = module._state
        self._lr = float(state.learning_rate) if state.learning_rate is not None else 1e-3
        if self._kind == "AdamW":
            for group in ("momentum0", "momentum1"):
                held = state.optimizer.setdefault(group, {})
                for p in module.parameters():
                    if p.requires_grad:
                        held[p.name] = held[p.name].to(module._device) if p.name in held else torch.zeros_like(p.data)

    def set_learning_rate(self, lr: float) -> None:
        self._lr = float(lr)
        self._module._state.learning_rate = self._lr

    def get_learning_rate(self) -> float:
        return self._lr

    def step(self) -> None:
        state = self._module._state
        params = [p for p in self._module.parameters() if p.requires_grad]
        state.optimizer_step += 1
        names = ["learning_rate"]
        values: List[object] = [torch.tensor([self._lr], dtype=torch.float32)]
        if self._kind == "AdamW":
            names.append("step")
            values.append(torch.tensor([state.optimizer_step], dtype=torch.int64))
        names += ["params", "gradients"]
        values += [[p.data for p in params], [p.grad for p in params]]
        if self._kind == "AdamW":
            names += ["first_order_moments", "second_order_moments"]
            values += [[state.optimizer["momentum0"][p.name] for p in params], [state.optimizer["momentum1"][p.name] for p in params]]
        with torch.no_grad():
            self._sess._sess.run(self._C.RunOptions(), names, values, ["updated_flag"])


class LinearLRScheduler:
    """Linear warm-up to the initial rate, then linear decay to zero at ``total_step_count``."""

    def __init__(self, optimizer: Optimizer, warmup_step_count: int, total_step_count: int, initial_lr: Optional[float] = None):
        self._opt, self._warm, self._total = optimizer, int(warmup_step_count), int(total_step_count)
        self._base = float(initial_lr) if initial_lr is not None else optimizer.get_learning_rate()
        self._step = 0
        self._apply()

    def _apply(self) -> None:
        s = self._step
        if s < self._warm:
            f = s / max(1, self._warm)
        else:
            f = max(0.0, (self._total - s) / max(1, self._total - self._warm))
        self._opt.set_learning_rate(self._base * f)

    def step(self) -> None:
        self._step += 1
        self._apply()
