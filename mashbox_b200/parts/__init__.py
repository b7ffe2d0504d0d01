"""Parts a layer is put together from.  Importing this package registers the built-in kinds."""
from . import (base, norm, position, conv, attention, diff_attention, latent_attention, channel_delta,  # noqa: F401
               feed_forward, routed_experts, token_side, block, embedding, retention, sigmoid_attention,
               side_by_side, gated_linear, ssd)
from .base import (PartSpec, LayerSpec, LayerRun, ModelSpec, Env, StepContext, StepInputs, Workspace,  # noqa: F401
                   register, make)
