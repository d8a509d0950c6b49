"""Data pipeline: sources, shards, iterators, codecs. The GPU-side preprocessing lives in the input operator."""
from .datasets import (Cifar10DataSource, DataSource, MnistDataSource, SyntheticDataSource, compute_mean,  # noqa: F401
                       open_data_file, open_split)
from .iterators import (AsyncPoolDataIter, AsyncQueueDataIter, AugmentDataSource, BatchIter,  # noqa: F401
                        CyclicEpisodeIterator, CyclicSampleDataIter, ParallelJoinDataIter, PartitionDataSource,
                        RaggedBatchIter, RandomEpisodeIterator, RandomIndexIter, RandomSampleDataIter, RangeDataShard, RangeWrapDataShard,
                        SampleIterator, SequentialSampleIter, TransformDataIter, cyclic_partition_shard,
                        episode_ranges, partition_shard)
