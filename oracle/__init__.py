"""CPU oracle for the fast-weight kernels: test infrastructure, never the product.

``kernels`` restates the reference's CUDA kernels (explicit forward and
backward recurrences); ``loops`` restates the reference's per-timestep PyTorch
formulation (gradients by autograd).  Only the test-suite, the smoke check and
the benchmark's CPU legs may import this package.
"""
