"""twinkle_b200 — a Blackwell-native LLM training workbench.

Same public surface as modelscope/twinkle (``initialize``, ``remote_class``,
``DeviceMesh``, model / sampler / dataset / server components) on one parallel
engine whose hot paths are hand-written sm_100a kernels.
"""
from .version import __version__
from .utils.device_mesh import DeviceGroup, DeviceMesh
from .utils.platform import GPU, Platform
from .utils.logger import get_logger
from .utils.framework import Torch
from .infra import (get_device_placement, get_global_device_mesh, initialize, is_initialized, remote_class, remote_function,
                    shutdown)

__all__ = ['__version__', 'DeviceGroup', 'DeviceMesh', 'GPU', 'Platform', 'get_logger', 'Torch', 'initialize',
           'is_initialized', 'remote_class', 'remote_function', 'get_device_placement', 'get_global_device_mesh', 'shutdown']
