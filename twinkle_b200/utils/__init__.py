from .device_mesh import DeviceGroup, DeviceMesh, is_last_rank, is_master
from .framework import Torch
from .import_utils import exists, requires
from .loader import Plugin, construct_class
from .logger import get_logger
from .network import find_free_port, find_node_ip
from .platform import GPU, Platform
from .seed import stable_seed
