"""Tensor / expert / pipeline parallel plumbing: one process per GPU, `torch.distributed`
for the control plane, peer memory for the fused compute+collective kernels."""
