"""Command-line tools: ``perf_test`` (latency / throughput of a model) and ``onnx_test_runner`` (ONNX test-data
directories), the counterparts of onnxruntime/test/perftest and onnxruntime/test/onnx."""
