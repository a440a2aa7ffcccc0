"""Sampler / scheduler catalogue with per-backend admission and name normalisation (the data behind `/v1/samplers`;
serenitymojo/sampling/sampler_registry.mojo:8-777)."""
from __future__ import annotations

import json
from typing import Dict, List, Optional, Tuple

SAMPLERS: Dict[str, Dict] = {
    "euler": {"family": "euler", "order": 1, "stochastic": False},
    "euler_ancestral": {"family": "euler", "order": 1, "stochastic": True},
    "heun": {"family": "heun", "order": 2, "stochastic": False},
    "dpmpp_2m": {"family": "dpmpp", "order": 2, "stochastic": False},
    "dpmpp_2m_sde": {"family": "dpmpp", "order": 2, "stochastic": True},
    "dpmpp_sde": {"family": "dpmpp", "order": 2, "stochastic": True},
    "uni_pc": {"family": "unipc", "order": 2, "stochastic": False},
    "uni_pc_bh2": {"family": "unipc", "order": 2, "stochastic": False},
    "res_2s": {"family": "res", "order": 2, "stochastic": False},
    "res_2s_sde": {"family": "res", "order": 2, "stochastic": True},
    "lcm": {"family": "lcm", "order": 1, "stochastic": True},
    "ddim": {"family": "euler", "order": 1, "stochastic": False},
}
SCHEDULERS = ["simple", "normal", "karras", "exponential", "sgm_uniform", "beta", "linear_quadratic", "flux_shift",
              "qwen_shift", "ltx_token_shift", "distilled"]
_ALIASES = {"unipc": "uni_pc", "uni-pc": "uni_pc", "dpm++ 2m": "dpmpp_2m", "dpmpp2m": "dpmpp_2m", "dpm++_2m": "dpmpp_2m",
            "euler a": "euler_ancestral", "euler_a": "euler_ancestral", "res2s": "res_2s", "dpm++ 2m sde": "dpmpp_2m_sde"}

# which (sampler, scheduler) pairs each backend really implements; anything else is rejected before enqueue
ADMISSION: Dict[str, Dict[str, List[str]]] = {
    "flux": {"samplers": ["euler"], "schedulers": ["simple", "flux_shift"]},
    "klein": {"samplers": ["euler"], "schedulers": ["simple", "flux_shift"]},
    "zimage": {"samplers": ["euler", "dpmpp_2m", "uni_pc"], "schedulers": ["simple", "sgm_uniform"]},
    "qwenimage": {"samplers": ["euler", "uni_pc"], "schedulers": ["simple", "qwen_shift"]},
    "sd3": {"samplers": ["euler", "dpmpp_2m"], "schedulers": ["simple", "sgm_uniform"]},
    "sdxl": {"samplers": ["euler", "euler_ancestral", "dpmpp_2m", "uni_pc", "ddim"], "schedulers": ["normal", "karras", "simple"]},
    "ltx2": {"samplers": ["euler", "res_2s", "res_2s_sde"], "schedulers": ["linear_quadratic", "ltx_token_shift", "distilled"]},
    "stub": {"samplers": list(SAMPLERS), "schedulers": SCHEDULERS},
}


def normalize_sampler(name: str) -> str:
    n = name.strip().lower().replace("-", "_") if name else "euler"
    n = _ALIASES.get(n, _ALIASES.get(n.replace("_", " "), n))
    return n


def admit(backend: str, sampler: str, scheduler: str) -> Tuple[bool, str]:
    """(ok, reason). Unknown names and unsupported pairs fail loudly instead of silently falling back."""
    s = normalize_sampler(sampler)
    sch = (scheduler or "simple").strip().lower()
    if s not in SAMPLERS:
        return False, f"unknown sampler '{sampler}'"
    if sch not in SCHEDULERS:
        return False, f"unknown scheduler '{scheduler}'"
    adm = ADMISSION.get(backend)
    if adm is None:
        return False, f"unknown backend '{backend}'"
    if s not in adm["samplers"]:
        return False, f"sampler '{s}' is not implemented by backend '{backend}' (supported: {', '.join(adm['samplers'])})"
    if sch not in adm["schedulers"]:
        return False, f"scheduler '{sch}' is not implemented by backend '{backend}'"
    return True, ""


def registry_json() -> str:
    return json.dumps({"schema": "serenity.samplers.v1", "samplers": SAMPLERS, "schedulers": SCHEDULERS,
                       "admission": ADMISSION}, sort_keys=True)


def karras_sigmas(n: int, sigma_min: float, sigma_max: float, rho: float = 7.0) -> List[float]:
    out = []
    for i in range(n):
        t = i / max(n - 1, 1)
        out.append((sigma_max ** (1 / rho) + t * (sigma_min ** (1 / rho) - sigma_max ** (1 / rho))) ** rho)
    return out + [0.0]
