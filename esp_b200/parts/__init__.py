from .base import ParamSpec, Part, Runtime, StepContext, Workspace, build, register, walk
from . import attention, block, delta, embedding, ffn, latent_attention, norm, parallel, position, recurrent, selective  # noqa: F401  (fills the registries)

__all__ = ["ParamSpec", "Part", "Runtime", "StepContext", "Workspace", "build", "register", "walk"]
