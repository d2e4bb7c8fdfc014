from .gemm_allreduce import (gemm_k_split_allreduce, gemm_k_split_two_shot, gemm_n_split, shard_k, shard_n)
from .peer_memory import (CollectiveClock, MulticastSharedTensor, PeerSharedTensor, TileFusedAllreduce, TwoShotAllreduce,
                          slice_bounds)
