"""Loss registry.  Parity: reference ``src/twinkle/loss/__init__.py:12-33``
(string → class table used by ``set_loss('GRPOLoss')`` and the CLI)."""
from .base import Loss
from .cross_entropy import (ChunkedCrossEntropyLoss, CrossEntropyLoss, DFTLoss, FusedLinearCrossEntropyLoss,
                            LigerFusedLinearCrossEntropyLoss, MSELoss)
from .dpo import CPOLoss, DPOLoss, ORPOLoss, SimPOLoss
from .gkd import GKDLoss
from .grpo import BNPOLoss, CISPOLoss, DRGRPOLoss, GRPOLoss, GSPOLoss, SAPOLoss
from .infonce import InfonceLoss

torch_loss_mapping = {
    'cross_entropy': CrossEntropyLoss, 'dft': DFTLoss, 'chunked_cross_entropy': ChunkedCrossEntropyLoss,
    'fused_linear_cross_entropy': FusedLinearCrossEntropyLoss, 'mse': MSELoss, 'grpo': GRPOLoss, 'gspo': GSPOLoss,
    'sapo': SAPOLoss, 'cispo': CISPOLoss, 'bnpo': BNPOLoss, 'dr_grpo': DRGRPOLoss, 'dpo': DPOLoss, 'simpo': SimPOLoss,
    'cpo': CPOLoss, 'orpo': ORPOLoss, 'gkd': GKDLoss, 'infonce': InfonceLoss,
}
for _c in list(torch_loss_mapping.values()):
    torch_loss_mapping[_c.__name__] = _c
torch_loss_mapping['LigerFusedLinearCrossEntropyLoss'] = FusedLinearCrossEntropyLoss
torch_loss_mapping['liger_fused_linear_cross_entropy'] = FusedLinearCrossEntropyLoss  # the reference's registry key for the same loss

__all__ = ['Loss', 'torch_loss_mapping'] + sorted({c.__name__ for c in torch_loss_mapping.values()})
