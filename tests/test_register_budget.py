"""The exchange kernels must fit on an SM beside a resident CTA of the tensor-core kernel.

The gradient exchange overlaps the backward pass only if a 128-thread block of `allreduce_sgd_kernel` / `ar_push_kernel`
finds room in the register file next to the 352-thread CTA of `gemm_tc_kernel` that occupies every SM. Registers are
handed out in units of 8 per thread to whole warps, four warps at a time; an SM has 65536: the CTA's 11 warps count as
12, so at 144 registers it takes 55296 and leaves exactly the 10240 of an exchange block (4 warps x 80). A change that
pushes the tensor-core kernel past 144 registers per thread silently serialises exchange and backward (measured: +15 % step time on 2 GPUs), so the
compiler's report is checked here. Needs nvcc, no GPU."""
import os
import re
import shutil
import subprocess

import pytest

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "rembrandt_b200", "csrc")
SM_REGISTERS = 65536
GEMM_THREADS, COMM_THREADS = 352, 128


def _registers(source, fast_math):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xptxas", "-v", "-I", CSRC, "-c",
           os.path.join(CSRC, source), "-o", os.devnull] + (["--use_fast_math"] if fast_math else [])
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    regs, name = {}, None
    for line in out.stderr.splitlines():
        m = re.search(r"Compiling entry function '(\S+)'", line)
        if m:
            name = m.group(1)
        m = re.search(r"Used (\d+) registers", line)
        if m and name:
            regs[name] = max(regs.get(name, 0), int(m.group(1)))
            name = None
    return regs


def _per_block(regs_per_thread, threads):
    """Registers a block takes: 8-register units per thread, whole warps, warps handed out four at a time."""
    warps = ((threads + 31) // 32 + 3) // 4 * 4
    return (regs_per_thread + 7) // 8 * 8 * 32 * warps


def test_exchange_blocks_fit_beside_a_tensor_core_cta():
    gemm = _registers("gemm_tc.cu", fast_math=True)
    comm = _registers("comm_p2p.cu", fast_math=False)
    gemm_regs = max(v for k, v in gemm.items() if "gemm_tc_kernel" in k)
    wanted = [k for k in comm if "allreduce_sgd_kernel" in k or "ar_push_kernel" in k or "ar_wait_kernel" in k]
    assert len(wanted) == 3, sorted(comm)
    for k in wanted:
        need = _per_block(gemm_regs, GEMM_THREADS) + _per_block(comm[k], COMM_THREADS)
        assert need <= SM_REGISTERS, (f"{k}: {comm[k]} registers x {COMM_THREADS} threads do not fit beside gemm_tc_kernel "
                                      f"({gemm_regs} x {GEMM_THREADS}): {need} > {SM_REGISTERS}")
