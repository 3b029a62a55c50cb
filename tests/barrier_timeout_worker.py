"""Worker of tests/test_failure_gpu.py: a peer that never joins a flag barrier makes the wait run out, the kernel
returns a status, the host raises, and the CUDA context stays usable. Nothing faults or hangs: the absent rank
simply waits on the host for the other one to finish."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    out_path = sys.argv[1]
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    dev = torch.device("cuda", torch.cuda.current_device())
    from tunix_b200 import _lib
    from tunix_b200.ops import kernels as K
    from tunix_b200.parallel import symm
    bar = symm.SymmBarrier(dev, timeout_ms=500)
    store = dist.distributed_c10d._get_default_store()
    bar.wait()                                   # both ranks: completes
    torch.cuda.synchronize()
    _lib.raise_if_kernel_error()
    res = {}
    if rank == 0:
        bar.wait()                               # rank 1 never posts this epoch
        torch.cuda.synchronize()
        try:
            _lib.raise_if_kernel_error()
            res["raised"] = False
        except RuntimeError as e:
            res["raised"], res["message"] = True, str(e)
        a = torch.randn(256, 256, device=dev).to(torch.bfloat16)
        c = K.gemm(a, a)                         # the context still works
        torch.cuda.synchronize()
        _lib.raise_if_kernel_error()
        res["usable"] = bool(torch.isfinite(c.float()).all())
        json.dump(res, open(out_path, "w"))
        store.set("rank0_done", "1")
    else:
        store.wait(["rank0_done"])               # between steps, nothing in flight on this GPU
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
