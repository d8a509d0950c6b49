"""rembrandt_b200: a Blackwell-native (sm_100a) convolutional-network training framework.

Layers (top to bottom): ``cli`` entry points, ``models`` (descriptors, builders, templates, the network
container), ``optim`` + ``trainer`` (SGD rules, schedules, the training loop), ``parallel`` (communication
backends), ``ops`` (operator library over hand-written CUDA kernels), ``data`` (input pipeline), ``utils``
(blob codec, checkpoints, RNG, logging) and the native libraries under ``csrc``.
"""
__version__ = "0.1.0"
