"""Model registry: family name -> constructor of the module that sits between the embedding
and the final norm. (Behavioural reference: ironcore/models/__init__.py:14-25.)"""

from .families import FAMILIES, family_of, resolve_family_defaults
from .language_model import IGNORE_INDEX, LanguageModel, get_model_dtype, masked_mean_loss


def get_model_provider_func(config):
    """Return a callable building the body for ``config.model.name`` (transformer or dummy)."""
    fam = family_of(config.model.name)
    if fam == "DUMMY":
        from .dummy import DummyModel

        return DummyModel
    from .transformer import TransformerModel

    return TransformerModel


__all__ = ["FAMILIES", "IGNORE_INDEX", "LanguageModel", "family_of", "get_model_dtype", "get_model_provider_func",
           "masked_mean_loss", "resolve_family_defaults"]
