"""CUDA sources for sm_100a, their build step and their ctypes bindings."""
