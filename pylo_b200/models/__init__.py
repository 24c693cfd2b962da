from .Meta_MLP import MetaMLP
from .CELO2_MLP import CELO2MLP, CELO2_FEATURE_DIMS
from .VeLO_MLP import VeLOMLP
from .VeLO_RNN import VeLORNN

__all__ = ["MetaMLP", "CELO2MLP", "CELO2_FEATURE_DIMS", "VeLOMLP", "VeLORNN"]
