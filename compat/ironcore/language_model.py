"""``LanguageModel(config, loss_fn)`` (reference: ironcore/language_model.py:21-234)."""

from ironcore_b200.models.language_model import LanguageModel  # noqa: F401
