"""Select the native build and the CUDA device the operators run on.

The reference chooses between two Ascend kernel packages by asking ``npu-smi`` (python/ops_gnn/_device.py:15-44 of
ops-gnn).  This build ships one package for NVIDIA B200 (sm_100a); selection only answers "which directory holds
``_pybind.so``" and, when CUDA is up, refuses devices the kernels were not compiled for.
"""
import os

SUPPORTED_TARGETS = ("sm100",)
_COMPUTE_CAPABILITY = (10, 0)


def select_target() -> str:
    """Return the package sub-directory that holds the native libraries.

    ``OPS_GNN_TARGET`` overrides detection (only ``sm100`` exists).  With CUDA initialised the current device, or the
    one named by ``OPS_GNN_DEVICE``, must report compute capability 10.0; without a visible GPU (build machines) the
    only target is returned so that the extension can still be imported and inspected.
    """
    override = os.getenv("OPS_GNN_TARGET", "").lower()
    if override:
        if override not in SUPPORTED_TARGETS:
            raise ValueError("OPS_GNN_TARGET must be sm100")
        return override
    import torch

    if not torch.cuda.is_available():
        return "sm100"
    index = os.getenv("OPS_GNN_DEVICE")
    device = int(index) if index not in (None, "") else torch.cuda.current_device()
    if device < 0 or device >= torch.cuda.device_count():
        raise RuntimeError(f"OPS_GNN_DEVICE={device} is not a visible CUDA device")
    capability = torch.cuda.get_device_capability(device)
    if capability != _COMPUTE_CAPABILITY:
        raise RuntimeError(
            f"Unsupported CUDA device {torch.cuda.get_device_name(device)!r} (compute capability "
            f"{capability[0]}.{capability[1]}); this build contains sm_100a kernels only")
    return "sm100"
