"""Samplers: flow-matching and DDPM-family schedules, multistep solvers, guidance, sampler registry."""
from . import ddpm, guidance, inpaint, ltx2, multistep, registry
from .flow_match import *  # noqa: F401,F403
