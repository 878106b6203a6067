"""gnn_benchmark_b200: B200-native distributed graph aggregation (SpMM + quantised halo exchange).

The reference's Python-facing names (Aggregator, SPMM_forward/SPMM_backward, Communicator,
Quantizer_for_all_procs, CommSplits, CommBuffer, DistributedGraph[ForPre], load_data,
TimeRecorder) over hand-written sm_100a CUDA kernels behind the C ABI of include/gnnagg.h.
"""
from .sparse import SparseTensor
from .spmm_kernel import SPMM_forward, SPMM_backward, build_plan
from .quantizer import QuantizerForPureBits, QuantizerForMixedBits, Quantizer_for_all_procs
from .time_recorder import TimeRecorder
from .data_manager import (CommBuffer, CommBufferForQuantization, CommSplits, DistributedGraph,
                           DistributedGraphForPre, DataProcessor, DataProcessorForPreAggresive, load_data)
from .communicator import Communicator
from .assigner import Assigner
from .aggregator import Aggregator

__all__ = [
    "SparseTensor", "SPMM_forward", "SPMM_backward", "build_plan", "QuantizerForPureBits", "QuantizerForMixedBits",
    "Quantizer_for_all_procs", "TimeRecorder", "CommBuffer", "CommBufferForQuantization", "CommSplits",
    "DistributedGraph", "DistributedGraphForPre", "DataProcessor", "DataProcessorForPreAggresive", "load_data",
    "Communicator", "Aggregator", "Assigner",
]
