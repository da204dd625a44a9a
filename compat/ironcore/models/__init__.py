"""Model registry (reference: ironcore/models/__init__.py:14-25)."""

from ironcore_b200.models import get_model_provider_func  # noqa: F401

from .dummy import DummyModel  # noqa: F401
from .transformer import TransformerLayer, TransformerModel  # noqa: F401
