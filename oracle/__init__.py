"""Test infrastructure: CPU restatement of the reference's resampling path and a loader for
the reference's own CUDA kernels.  Nothing in the shipped package imports this."""
