"""``hmf env``: versions of the pieces this framework runs on."""
import os
import platform


def get_env() -> dict:
    info = {"python": platform.python_version(), "platform": platform.platform()}
    try:
        import torch
        info["torch"] = torch.__version__
        info["cuda_available"] = torch.cuda.is_available()
        if torch.cuda.is_available():
            info["gpu"] = torch.cuda.get_device_name(0)
            info["gpu_count"] = torch.cuda.device_count()
            info["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
    except Exception as e:  # pragma: no cover
        info["torch"] = f"unavailable ({e})"
    from ..ops import _lib
    info["kernel_library"] = str(_lib._KERNELS_PATH) if _lib.kernels_available() else "not built"
    for k in ("NNODES", "NODE_RANK", "NPROC_PER_NODE", "MASTER_ADDR", "MASTER_PORT", "HMF_VERBOSITY"):
        if k in os.environ:
            info[k] = os.environ[k]
    return info


def print_env() -> None:
    for k, v in get_env().items():
        print(f"- {k}: {v}")
