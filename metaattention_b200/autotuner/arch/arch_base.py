class Arch:
    """Static facts about one GPU model."""

    name = "base"
    platform = "CUDA"
    compute_capability = "unknown"
    compute_max_core = 0          # number of SMs
    smem_cap = 0                  # bytes of shared memory per CTA
    reg_cap = 65536               # 32-bit registers per SM
    register_per_thread = 255
    warp_size = 32
    sm_partition = 4
    threads_cap = 1024
    tmem_columns = 0              # tensor-memory columns per SM (0 = none)
    hbm_gbs = 0.0                 # nominal HBM bandwidth, GB/s
    bf16_tflops = 0.0             # nominal dense bf16 tensor throughput, TFLOP/s

    def __repr__(self):
        return f"<{self.name} sm_{self.compute_capability}>"
