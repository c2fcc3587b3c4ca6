"""cuda_sm100: lowers annotated loops onto hand-written CUDA C templates (NVRTC, sm_100a)."""
