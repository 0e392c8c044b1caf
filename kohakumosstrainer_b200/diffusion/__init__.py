"""Rectified-flow objective, timestep samplers and the Euler + CFG sampler."""

from .objective import LOSSES, WEIGHTINGS, TokenNormalizer, noise_latents, token_loss
from .sampling import SampleResult, initial_noise, latent_grid, moss_sigmas, sample_latents, unpack
from .timestep import TIMESTEPS, LogitNormalTimestep, MossTimestep, UniformTimestep, shift_sigma

__all__ = [
    "LOSSES", "WEIGHTINGS", "TokenNormalizer", "noise_latents", "token_loss", "SampleResult", "initial_noise",
    "latent_grid", "moss_sigmas", "sample_latents", "unpack", "TIMESTEPS", "LogitNormalTimestep", "MossTimestep",
    "UniformTimestep", "shift_sigma",
]
