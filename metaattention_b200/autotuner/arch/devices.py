from .arch_base import Arch


class A100(Arch):
    name = "A100"
    compute_capability = "80"
    compute_max_core = 108
    smem_cap = 163 * 1024
    hbm_gbs = 2039.0
    bf16_tflops = 312.0


class RTX4090(Arch):
    name = "RTX4090"
    compute_capability = "89"
    compute_max_core = 128
    smem_cap = 99 * 1024
    hbm_gbs = 1008.0
    bf16_tflops = 165.0


class H100(Arch):
    name = "H100"
    compute_capability = "90a"
    compute_max_core = 132
    smem_cap = 227 * 1024
    hbm_gbs = 3350.0
    bf16_tflops = 989.0


class B200(Arch):
    name = "B200"
    compute_capability = "100a"
    compute_max_core = 148
    smem_cap = 227 * 1024
    tmem_columns = 512
    hbm_gbs = 7700.0
    bf16_tflops = 2250.0
