"""Stand-ins for two pure-Python dependencies of the reference that the offline image lacks.

The reference package under ``baseline/_ref`` stays byte-for-byte unmodified.  Its import chain touches
``draccus`` (config codec: choice registries, encode / decode hooks, CLI wrapping) and ``accelerate`` (launcher
object and seeding helper).  Neither takes part in the measured training step: the benchmark builds the policy
config as a plain dataclass and drives ``PI05Policy.forward`` -> ``backward`` -> ``MasterWeightOptimizer.step``
directly.  Only the names the import chain and that step touch are provided; anything else raises.
``install()`` returns the list of stand-ins it registered so the bench line can disclose them.
"""

from __future__ import annotations

import functools
import importlib
import importlib.machinery
import random
import sys
import types


def _has(name: str) -> bool:
    try:
        importlib.import_module(name)
        return True
    except Exception:
        return False


class _HookTable:
    """``draccus.encode`` / ``draccus.decode``: callable with a ``register`` hook (registrations are kept, unused)."""

    def __init__(self, name):
        self._name, self.registry = name, {}

    def register(self, cls, fn=None, include_subclasses=False):
        if fn is None:
            def deco(f):
                self.registry[cls] = f
                return f
            return deco
        self.registry[cls] = fn
        return fn

    def __call__(self, *a, **k):
        raise NotImplementedError(f"draccus.{self._name} stand-in: the config codec is not part of the timed step")


def _make_draccus() -> types.ModuleType:
    m = types.ModuleType("draccus")
    m.__stand_in__ = True
    m.CHOICE_TYPE_KEY = "type"

    class ChoiceRegistry:
        """Base class of the reference's config families: keeps name -> subclass per registry root."""

        @classmethod
        def _registry(cls):
            for base in cls.__mro__:
                if "_choice_registry" in base.__dict__:
                    return base.__dict__["_choice_registry"]
            # the first class below ChoiceRegistry in the MRO owns the table
            roots = [b for b in cls.__mro__ if ChoiceRegistry in b.__bases__]
            root = roots[-1] if roots else cls
            root._choice_registry = {}
            return root._choice_registry

        @classmethod
        def register_subclass(cls, name, *a, **k):
            def deco(sub):
                cls._registry()[name] = sub
                sub._choice_name = name
                return sub
            return deco

        @classmethod
        def get_choice_class(cls, name):
            return cls._registry()[name]

        @classmethod
        def get_known_choices(cls):
            return dict(cls._registry())

        @classmethod
        def get_choice_name(cls, sub):
            for k, v in cls._registry().items():
                if v is sub:
                    return k
            return getattr(sub, "_choice_name", sub.__name__)

    m.ChoiceRegistry = ChoiceRegistry
    m.encode, m.decode = _HookTable("encode"), _HookTable("decode")

    def _unavailable(name):
        def fn(*a, **k):
            raise NotImplementedError(f"draccus.{name} stand-in: the config codec is not part of the timed step")
        fn.__name__ = name
        return fn

    for name in ("parse", "load", "dump"):
        setattr(m, name, _unavailable(name))
    m.set_config_type = lambda *_a, **_k: None

    class _ConfigType:
        def __init__(self, *_a):
            pass

        def __enter__(self):
            return self

        def __exit__(self, *exc):
            return False

    m.config_type = _ConfigType

    def wrap(*_a, **_k):
        def deco(fn):
            @functools.wraps(fn)
            def inner(*a, **k):
                return fn(*a, **k)
            return inner
        return deco

    m.wrap = wrap
    parsers = types.ModuleType("draccus.parsers")
    encoding = types.ModuleType("draccus.parsers.encoding")
    encoding.encode = m.encode
    decoding = types.ModuleType("draccus.parsers.decoding")
    decoding.decode = m.decode
    parsers.encoding, parsers.decoding = encoding, decoding
    m.parsers = parsers
    utils = types.ModuleType("draccus.utils")
    utils.DecodingError = type("DecodingError", (Exception,), {})
    utils.ParsingError = type("ParsingError", (Exception,), {})
    m.utils = utils
    sys.modules.update({"draccus": m, "draccus.parsers": parsers, "draccus.parsers.encoding": encoding,
                        "draccus.parsers.decoding": decoding, "draccus.utils": utils})
    return m


def _make_accelerate() -> types.ModuleType:
    m = types.ModuleType("accelerate")
    m.__stand_in__ = True
    m.__spec__ = importlib.machinery.ModuleSpec("accelerate", None)

    class Accelerator:  # only referenced in annotations / isinstance checks on the imported paths
        def __init__(self, *a, **k):
            raise NotImplementedError("accelerate.Accelerator stand-in: the benchmark drives the step directly")

    m.Accelerator = Accelerator
    utils = types.ModuleType("accelerate.utils")

    def set_seed(seed, device_specific=False, deterministic=False):
        import numpy as np
        import torch
        random.seed(seed), np.random.seed(seed), torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    utils.set_seed = set_seed
    for name in ("DistributedDataParallelKwargs", "DistributedType", "DeepSpeedPlugin", "FullyShardedDataParallelPlugin"):
        setattr(utils, name, type(name, (), {}))
    utils.gather_object = lambda obj: obj
    utils.broadcast_object_list = lambda objs, from_process=0: objs
    m.utils = utils
    m.PartialState = type("PartialState", (), {})
    sys.modules.update({"accelerate": m, "accelerate.utils": utils})
    return m


class _AbsentModule(types.ModuleType):
    """A module that is imported by the reference at file scope but never used on the measured path: every
    attribute is a fresh placeholder class (usable as a base class or in an annotation) whose construction raises."""

    def __getattr__(self, attr):
        if attr.startswith("__"):
            raise AttributeError(attr)
        full = f"{self.__name__}.{attr}"

        def _init(self, *a, **k):
            raise NotImplementedError(f"{full} stand-in: not available offline and not part of the timed step")

        cls = type(attr, (), {"__init__": _init, "__module__": self.__name__})
        setattr(self, attr, cls)
        return cls


def _make_absent(name: str, submodules: tuple[str, ...] = ()) -> None:
    m = _AbsentModule(name)
    m.__stand_in__ = True
    m.__path__ = []
    m.__spec__ = importlib.machinery.ModuleSpec(name, None, is_package=True)
    sys.modules[name] = m
    for sub in submodules:
        sm = _AbsentModule(f"{name}.{sub}")
        sm.__path__ = []
        sm.__spec__ = importlib.machinery.ModuleSpec(f"{name}.{sub}", None, is_package=True)
        sys.modules[f"{name}.{sub}"] = sm
        setattr(m, sub.split(".")[0], sys.modules[f"{name}.{sub.split('.')[0]}"])


# file-scope imports of the reference that the image lacks and the training step never calls
_ABSENT = {
    "jsonlines": (),
    "deepdiff": (),
    "termcolor": (),
    "av": ("video", "video.frame"),
    "torchcodec": ("decoders",),
    "gymnasium": ("spaces", "vector", "envs", "envs.registration", "wrappers"),
    "imageio": ("v2",),
}


def _warm_transformers() -> None:
    """Imports the transformers modules the reference uses BEFORE any stand-in exists, so that transformers'
    own optional-dependency probes (accelerate, torchcodec, av ...) see the image as it really is."""
    import transformers  # noqa: F401
    for name in ("transformers.models.gemma.modeling_gemma", "transformers.models.gemma3.modeling_gemma3",
                 "transformers.models.paligemma.modeling_paligemma", "transformers.models.siglip.modeling_siglip",
                 "transformers.models.qwen3_vl.modeling_qwen3_vl", "transformers.models.auto",
                 "transformers.modeling_outputs", "transformers.tokenization_utils_base",
                 "transformers.integrations.deepspeed", "transformers.processing_utils"):
        try:
            importlib.import_module(name)
        except Exception:
            pass
    from transformers import AutoProcessor, AutoTokenizer, PreTrainedTokenizerFast  # noqa: F401


def _transformers_compat() -> list[str]:
    """The reference is written against transformers 4.5x; the image has 5.x.  Restores, on the library's classes,
    the 4.x attribute aliases that 5.x dropped and the reference reads.  Returns what was added."""
    added = []
    from transformers.models.paligemma.modeling_paligemma import PaliGemmaForConditionalGeneration as PG
    for alias in ("vision_tower", "language_model", "multi_modal_projector"):
        if not hasattr(PG, alias):
            setattr(PG, alias, property(lambda self, _a=alias: getattr(self.model, _a)))
            added.append(f"transformers-4.x alias PaliGemmaForConditionalGeneration.{alias}")
    return added


def install() -> list[str]:
    """Registers a stand-in for every missing dependency; returns their names (empty when the real ones import)."""
    made = []
    _warm_transformers()
    made += _transformers_compat()
    if not _has("draccus"):
        _make_draccus()
        made.append("draccus")
    if not _has("accelerate"):
        _make_accelerate()
        made.append("accelerate")
    for name, subs in _ABSENT.items():
        if not _has(name):
            _make_absent(name, subs)
            made.append(name)
    return made
