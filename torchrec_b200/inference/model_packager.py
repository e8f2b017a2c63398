"""Packaging a ``PredictFactory`` into one file a server can load (``torchrec/inference/model_packager.py:49``).

The package is a zip written by ``torch.package``: the pickled factory, its source modules (everything outside the interned
prefixes is taken from the serving environment), text / pickle configs, and the metadata the batching runtime reads."""
from __future__ import annotations

import abc
import pickle
from pathlib import Path
from typing import Any, BinaryIO, Dict, List, Optional, Type, TypeVar, Union

import torch
from torch.package import PackageExporter, PackageImporter

from torchrec_b200.inference.modules import PredictFactory

T = TypeVar("T")
_CONFIG_PACKAGE = "__configs"
_FACTORY_PACKAGE = "__predict_factory"

try:
    # the loader of a package exposes its importer to packaged code through this hook
    from torch.package import importer as _pkg_importer  # noqa: F401
except Exception:  # pragma: no cover
    _pkg_importer = None

_ACTIVE_IMPORTER: Optional[PackageImporter] = None


def load_config_text(name: str) -> str:
    assert _ACTIVE_IMPORTER is not None, "configs can only be read while a package is being loaded"
    return _ACTIVE_IMPORTER.load_text(_CONFIG_PACKAGE, name)


def load_pickle_config(name: str, clazz: Type[T]) -> T:
    assert _ACTIVE_IMPORTER is not None, "configs can only be read while a package is being loaded"
    loaded = _ACTIVE_IMPORTER.load_pickle(_CONFIG_PACKAGE, name)
    assert isinstance(loaded, clazz), f"the config {name} should be of type {clazz} but got {type(loaded)}"
    return loaded


class PredictFactoryPackager:
    """Subclass and name the modules that stay outside the package (``set_extern_modules``) or are replaced by stubs
    (``set_mocked_modules``); everything else the factory imports is stored inside."""

    @classmethod
    @abc.abstractmethod
    def set_extern_modules(cls, pe: PackageExporter) -> None:
        ...

    @classmethod
    @abc.abstractmethod
    def set_mocked_modules(cls, pe: PackageExporter) -> None:
        ...

    @classmethod
    def save_predict_factory(cls, predict_factory: Type[PredictFactory], configs: Dict[str, Any], output: Union[str, Path, BinaryIO],
                             extra_files: Dict[str, Union[str, bytes]], loader_code: str = "import %PACKAGE%\n\nMODULE_FACTORY=%PACKAGE%.%CLASS%\n",
                             package_importer: Any = None) -> None:
        kw = {"importer": package_importer} if package_importer is not None else {}
        with PackageExporter(output, **kw) as pe:
            cls.set_extern_modules(pe)
            cls.set_mocked_modules(pe)
            pe.extern(["sys"])
            pe.intern("**")
            for k, v in extra_files.items():
                if isinstance(v, str):
                    pe.save_text("extra_files", k, v)
                elif isinstance(v, bytes):
                    pe.save_binary("extra_files", k, v)
                else:
                    raise ValueError(f"Unsupported type {type(v)}")
            cls._save_predict_factory(pe, predict_factory, configs, loader_code=loader_code)

    @classmethod
    def _save_predict_factory(cls, pe: PackageExporter, predict_factory: Type[PredictFactory], configs: Dict[str, Any], loader_code: str) -> None:
        package_name, class_name = predict_factory.__module__, predict_factory.__name__
        pe.save_text(_FACTORY_PACKAGE, "loader.py", loader_code.replace("%PACKAGE%", package_name).replace("%CLASS%", class_name))
        pe.save_text(_FACTORY_PACKAGE, "factory_name", f"{package_name}:{class_name}")
        pe.save_source_string(f"{_FACTORY_PACKAGE}.__init__", "")
        for name, config in configs.items():
            if isinstance(config, str):
                pe.save_text(_CONFIG_PACKAGE, name, config)
            else:
                pe.save_pickle(_CONFIG_PACKAGE, name, config)
        pe.save_pickle(_FACTORY_PACKAGE, _FACTORY_PACKAGE, predict_factory)


def load_predict_factory(path: Union[str, Path, BinaryIO]) -> PredictFactory:
    """Instantiate the packaged factory class (its constructor may read configs through :func:`load_config_text`)."""
    global _ACTIVE_IMPORTER
    pi = PackageImporter(path)
    _ACTIVE_IMPORTER = pi
    try:
        factory_cls = pi.load_pickle(_FACTORY_PACKAGE, _FACTORY_PACKAGE)
        return factory_cls()
    finally:
        _ACTIVE_IMPORTER = None
