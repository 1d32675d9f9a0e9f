"""Constants shared by the host code and the kernels (csrc/common.cuh holds the same values)."""

PAGE = 64      # positions per cache page (WPC_PAGE)
