"""In-kernel communication over NVLink peer memory (symmetric buffers, flag barriers, fused
optimizer-step kernels). NCCL stays the bootstrap (handle exchange) and the fallback."""
