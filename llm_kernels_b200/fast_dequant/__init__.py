"""Mirror of the reference's fast_dequant/ folder: weight-only int4 kernels."""
