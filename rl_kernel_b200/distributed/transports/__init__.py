"""Transports under the fixed-order collectives: torch.distributed all-gather (NCCL or Gloo)
and CUDA symmetric memory over NVLink (``symm``)."""
