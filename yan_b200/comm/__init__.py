from .gemm_allreduce import (gemm_k_split_allreduce, gemm_n_split, shard_k, shard_n)
