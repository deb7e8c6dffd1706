from .comm import Communicator
from .fsdp import FSDPEngine
