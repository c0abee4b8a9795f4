"""Architecture families, one module each; importing this package registers them."""

from mlx_omnia_b200.architectures import bobarax, dolutar, fokalorn, muse_glimmer, narezen  # noqa: F401
