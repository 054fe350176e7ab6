"""onnxruntime_b200: a Blackwell-native (sm_100a) ONNX inference engine.

The public API mirrors ``onnxruntime``::

    import onnxruntime_b200 as ort
    sess = ort.InferenceSession("model.onnx", providers=["CUDAExecutionProvider"])
    outputs = sess.run(None, {"input": array})

The native runtime (``_core``) and the kernel library (``lib/libortb200_kernels.so``)
are built in-tree by ``python -m onnxruntime_b200.build``.
"""
__version__ = "0.1.0"

import os as _os

_here = _os.path.dirname(_os.path.abspath(__file__))
_built = any(f.startswith("_core") and f.endswith(".so") for f in _os.listdir(_here))

if _built:
    import torch as _torch  # noqa: F401  (loads libtorch before the extension)

    from .capi import *  # noqa: F401,F403
    from .capi import (  # noqa: F401
        EPFail, EngineError, Fail, InvalidArgument, InvalidGraph, InvalidProtobuf, ModelLoaded, NoModel, NoSuchFile,
        NotImplemented, OrtException, RuntimeException,
    )
else:
    # The package stays importable so that `python -m onnxruntime_b200.build` can run; everything else
    # fails loudly until the native runtime exists.
    def __getattr__(name):
        raise ImportError("onnxruntime_b200._core is not built: run `python -m onnxruntime_b200.build`")
