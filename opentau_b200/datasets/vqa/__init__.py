from .base import VQA_REGISTRY, VQADataset, make_vqa_dataset, register_vqa_dataset
from . import dummy, local  # noqa: F401  (registration side effects)

__all__ = ["VQADataset", "VQA_REGISTRY", "register_vqa_dataset", "make_vqa_dataset"]
