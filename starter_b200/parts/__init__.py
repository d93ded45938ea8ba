from .attention import GroupedQueryAttention
from .attention_diff import DifferentialAttention
from .attention_latent import LatentAttention
from .base import ROLES, ParamSpec, Part, Role, register_role, role_of
from .block import PreNormBlock
from .feedforward import BiasedFeedForward, GatedFeedForward, RoutedExperts
from .hyper import HyperConnection, HyperMixerOnlyBlock, HyperPreNormBlock, Pending
from .norm import RMSNorm
from .norm_dyt import DynamicTanh
from .registry import FAMILIES, lookup, register
from .rotary import InterleavedRotaryTable, Rotation, RotaryTable
from .sandwich import SandwichBlock, SandwichMixerOnlyBlock, Unsummed
from .wkv import WkvMixer

__all__ = ["FAMILIES", "ROLES", "Role", "register_role", "role_of", "GatedFeedForward", "GroupedQueryAttention", "DifferentialAttention", "DynamicTanh", "HyperConnection",
           "HyperMixerOnlyBlock", "HyperPreNormBlock", "Pending", "ParamSpec", "Part",
           "PreNormBlock", "RMSNorm", "RotaryTable", "Rotation", "lookup", "register", "BiasedFeedForward", "InterleavedRotaryTable", "LatentAttention", "RoutedExperts",
           "SandwichBlock", "SandwichMixerOnlyBlock", "Unsummed", "WkvMixer"]
