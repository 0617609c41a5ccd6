"""Host side of the specialised solver kernels (same module names as the
reference's ``instantmimic.utils.mjw_kernels``)."""
