from .moe import (BaseMoELayer, GroupedMLP, MoEAlltoAllTokenDispatcher, MoEAuxLossAutoScaler, MoELayer, MoELayerConfig,
                  MoERuntimeInputs, SharedExpertMLP, TopKRouter, z_loss_func)

__all__ = ["BaseMoELayer", "GroupedMLP", "MoEAlltoAllTokenDispatcher", "MoEAuxLossAutoScaler", "MoELayer",
           "MoELayerConfig", "MoERuntimeInputs", "SharedExpertMLP", "TopKRouter", "z_loss_func"]
