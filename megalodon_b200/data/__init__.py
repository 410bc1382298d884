"""Tokeniser and data loaders (`megalodon.data.tokenizer`, `megalodon.data.dataloader` in the reference);
the classes are also importable from the package itself."""
import importlib

_WHERE = {"Tokenizer": "tokenizer", "DataLoader": "dataloader", "SyntheticTokens": "dataloader"}
__all__ = sorted(_WHERE)


def __getattr__(name):
    if name in _WHERE:
        value = getattr(importlib.import_module(f"{__name__}.{_WHERE[name]}"), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
