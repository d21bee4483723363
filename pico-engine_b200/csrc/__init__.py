"""CUDA sources (sm_100a) and their build.  ``ops`` holds the Python side of every kernel."""
