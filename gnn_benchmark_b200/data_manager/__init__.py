"""Partition loading, communication-plan construction and exchange buffers.

Same module and class names as the reference's self_benchmark/a64fx/data_manager package."""
from .DistributedGraph import DistributedGraph
from .DistributedGraph import DistributedGraphForPre
from .CommBuffer import CommBuffer, CommBufferForQuantization
from .CommSplits import CommSplits
from .DataProcessor import DataProcessor, DataProcessorForPreAggresive
from .DataLoader import load_data, get_distributed_graph, get_distributed_graph_for_pre_aggressive
