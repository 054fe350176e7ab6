"""Benchmarks of the secondary configurations (BERT-large encoder, Mixtral-shaped MoE layer, int4 Llama-70B-shaped
decode layer).  Each prints one JSON line; each has a ``--baseline torch`` arm that runs the same math through
PyTorch's library kernels (cuBLAS, SDPA, NCCL) on the same box for comparison.  Run one process per GPU with
``python -m torch.distributed.run`` for more than one GPU."""
