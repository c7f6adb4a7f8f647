"""tips_b200: a Blackwell-native distributed-training framework with two
acceleration modes, collective communication and a sharded parameter server.

The public surface follows the reference's ``tips.tensorflow`` module
(tips/tensorflow/__init__.py, ops.py, functions.py) with PyTorch tensors in
place of TensorFlow ones.
"""
from .config import Config, get_config, set_config
from .runtime import (TipsError, barrier, init, initialized, is_initialized, local_rank, local_size, metrics, rank,
                      reset_collectives, shutdown, size)
from .parallel.collectives import (Average, Max, Min, Product, Sum, allgather, allgather_async, allreduce,
                                   allreduce_, allreduce_async, allreduce_async_, broadcast, broadcast_,
                                   broadcast_async, broadcast_async_, grouped_allreduce, poll, sparse_allreduce,
                                   synchronize)
from .parallel.compression import Compression
from .parallel.group import Group
from .parallel.optimizer import DistributedOptimizer
from .parallel.functions import (allgather_object, broadcast_object, broadcast_object_fn, broadcast_optimizer_state,
                                 broadcast_parameters, broadcast_variables, metric_average, allreduce_gradients,
                                 allreduce_value, allgather_value, broadcast_value, broadcast_global_variables,
                                 rank_op, size_op, local_rank_op, local_size_op)
from .parallel.tape import BroadcastGlobalVariablesHook, DistributedGradientTape

__version__ = "0.1.0"
from . import callbacks, elastic
from .utils.checkpoint import load_checkpoint, load_model, resume, save_checkpoint
