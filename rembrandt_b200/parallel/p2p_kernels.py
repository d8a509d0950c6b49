"""ctypes signatures of the peer-to-peer / multimem communication kernels (csrc/comm_p2p.cu)."""
SIGS = {}
