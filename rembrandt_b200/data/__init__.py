"""Data pipeline: sources, shards, iterators, codecs. The GPU-side preprocessing lives in the input operator."""
from .datasets import (Cifar10DataSource, DataSource, MnistDataSource, SyntheticDataSource, compute_mean,  # noqa: F401
                       open_data_file, open_split)
from .iterators import (AsyncPoolDataIter, AsyncQueueDataIter, BatchIter, CyclicSampleDataIter,  # noqa: F401
                        ParallelJoinDataIter, RandomSampleDataIter, RangeDataShard, RangeWrapDataShard,
                        SequentialSampleIter, TransformDataIter, cyclic_partition_shard, partition_shard)
