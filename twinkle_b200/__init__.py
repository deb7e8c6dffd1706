"""twinkle_b200 — a Blackwell-native LLM training workbench.

Same public surface as modelscope/twinkle (``initialize``, ``remote_class``,
``DeviceMesh``, model / sampler / dataset / server components) on one parallel
engine whose hot paths are hand-written sm_100a kernels.
"""
from .version import __release_datetime__, __version__
from .utils.device_mesh import DeviceGroup, DeviceMesh, is_master
from .utils.platform import GPU, Platform
from .utils.logger import get_logger
from .utils.framework import Torch
from .utils.import_utils import exists, requires
from .utils.loader import Plugin, check_unsafe, trust_remote_code
from .utils.network import find_free_port, find_node_ip
from .utils import framework as framework_util
from .utils import torch_utils as torch_util
from .infra import (get_device_placement, get_global_device_mesh, initialize, is_initialized, remote_class, remote_function,
                    shutdown)


def init_twinkle_client(*args, **kwargs):
    """``client.init_twinkle_client`` (imported on first use: the HTTP client stack is not needed for local training)."""
    from .client import init_twinkle_client as f
    return f(*args, **kwargs)


def init_tinker_client(*args, **kwargs):
    from .client import init_tinker_client as f
    return f(*args, **kwargs)


__all__ = ['__version__', '__release_datetime__', 'DeviceGroup', 'DeviceMesh', 'GPU', 'Platform', 'Plugin', 'get_logger', 'Torch', 'initialize',
           'is_initialized', 'is_master', 'remote_class', 'remote_function', 'get_device_placement', 'get_global_device_mesh', 'shutdown',
           'exists', 'requires', 'find_free_port', 'find_node_ip', 'trust_remote_code', 'check_unsafe', 'framework_util', 'torch_util',
           'init_twinkle_client', 'init_tinker_client']
