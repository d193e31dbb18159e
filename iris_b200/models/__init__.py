"""Model-level building blocks assembled from the fused operators (tensor-parallel decoder block)."""
