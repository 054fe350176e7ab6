"""Training on top of the inference runtime (the counterpart of the reference's ``orttraining`` tree).

* ``gradient_builder.build_gradient_graph``: forward ONNX graph -> graph with gradient outputs.
* ``artifacts.generate_artifacts``: training / eval / optimizer models and a checkpoint from a forward model
  (``orttraining/orttraining/python/training/artifacts.py``).
* ``api``: ``CheckpointState``, ``Module``, ``Optimizer``, ``LinearLRScheduler`` over those artifacts
  (``orttraining/orttraining/training_api``).
* ``megatron``: ``MegatronF`` / ``MegatronG`` and the column / row split of an MLP for tensor-parallel training.
* ``ORTModule``: a ``torch.nn.Module`` whose forward pass runs an ONNX graph in the native session and whose backward
  pass is the autograd tape recorded through the session's tensor-library kernels.
"""
from .gradient_builder import build_gradient_graph, supported_ops  # noqa: F401
from .ortmodule import ORTModule  # noqa: F401
from .artifacts import LossType, OptimType, generate_artifacts  # noqa: F401
from . import api  # noqa: F401
from . import megatron  # noqa: F401
