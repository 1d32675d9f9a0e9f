"""CUDA sources (sm_100a) and their in-tree build."""
