"""Partition loading, communication-plan construction and exchange buffers.

Same module and class names as the reference's self_benchmark/a64fx/data_manager package."""
from . import CommBuffer as _buffers
from . import CommSplits as _splits
from . import DataLoader as _loader
from . import DataProcessor as _plans
from . import DistributedGraph as _graphs

CommSplits = _splits.CommSplits
CommBuffer = _buffers.CommBuffer
CommBufferForQuantization = _buffers.CommBufferForQuantization
DistributedGraph = _graphs.DistributedGraph
DistributedGraphForPre = _graphs.DistributedGraphForPre
DataProcessor = _plans.DataProcessor
DataProcessorForPreAggresive = _plans.DataProcessorForPreAggresive
load_data = _loader.load_data
build_graph = _loader.build_graph
pad_feature_rows = _loader.pad_feature_rows
get_distributed_graph = _loader.get_distributed_graph
get_distributed_graph_for_pre_aggressive = _loader.get_distributed_graph_for_pre_aggressive

__all__ = [
    "CommSplits", "CommBuffer", "CommBufferForQuantization", "DistributedGraph", "DistributedGraphForPre",
    "DataProcessor", "DataProcessorForPreAggresive", "load_data", "build_graph", "pad_feature_rows",
    "get_distributed_graph", "get_distributed_graph_for_pre_aggressive",
]
