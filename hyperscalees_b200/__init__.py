"""B200-native EggRoll population step behind the HyperscaleES crate surface.

Sub-modules mirror the reference crates: `core` (hyperscalees-core), `noiser`
(hyperscalees-noiser), `models` (hyperscalees-models), `envs`
(hyperscalees-envs), `kernels` (hyperscalees-kernels + the oxide seam).  `ops`
holds the tensor-level wrappers over the C ABI (`include/hses.h`), `parallel` the
population sharding across GPUs, `data` the host-side MNIST readers, batch sampler
and CSV log of the trainer.
"""
from . import _lib  # noqa: F401

__all__ = ["core", "noiser", "models", "snn_transformer", "envs", "kernels", "ops", "parallel", "data"]
