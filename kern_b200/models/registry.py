"""Model families by name: ``name -> (config, manifest builder, synthetic-weights loader)``.

``kern run|bench|server --model NAME`` builds the manifest in memory and fills the weights with the family's
random-init checkpoint on the device (no files), which is how the benchmarks run without a network."""
from __future__ import annotations

import dataclasses


def families() -> dict:
    from . import dense, hybrid, latent, moe

    out = {}
    for cfg in (dense.TOY, dense.TINY, dense.DENSE_8B):
        out[cfg.name] = (cfg, dense.build_manifest, dense.load_random_weights, dense.random_weights)
    for cfg in (hybrid.TOY_HYBRID, hybrid.TINY_HYBRID, hybrid.TINY_HYBRID_K128, hybrid.HYBRID_27B):
        out[cfg.name] = (cfg, hybrid.build_manifest, hybrid.load_random_weights, hybrid.random_weights)
    for cfg in (moe.TOY_MOE, moe.TINY_MOE, moe.MOE_30B):
        out[cfg.name] = (cfg, moe.build_manifest, moe.load_random_weights, moe.random_weights)
    for cfg in (latent.TINY_LATENT, latent.TINY_LATENT_K128, latent.TINY_LATENT_MOE, latent.LATENT_48B):
        out[cfg.name] = (cfg, latent.build_manifest, latent.load_random_weights,
                         lambda cfg, **kw: latent.folded(cfg, latent.random_weights(cfg, **kw)))
    from . import toy_int

    for lined in (False, True):
        name = "toy-int-stateful" if lined else "toy-int"
        out[name] = (lined, lambda lined: toy_int.build_manifest(lined), lambda rt, cfg: None, lambda cfg: None)
    return out


def resolve(name: str, **overrides):
    """-> (config with overrides applied, builder, device loader, host weights maker)."""
    fam = families()
    if name not in fam:
        raise KeyError(f"unknown model `{name}`; known: {', '.join(sorted(fam))}")
    cfg, build, load, make = fam[name]
    overrides = {k: v for k, v in overrides.items() if v is not None}
    if not dataclasses.is_dataclass(cfg):
        return cfg, build, load, make          # a family without a config object (the integer model)
    return dataclasses.replace(cfg, **overrides), build, load, make
