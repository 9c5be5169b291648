"""Second-generation training stack: a data engine that indexes several datasets as one, a renderer from chat
samples to model inputs, a batch generator whose position can be saved and restored, and a trainer whose loss is
weighted by valid tokens over micro-batches and data-parallel ranks.  Counterpart of the reference's experimental
``hmf/v1`` package (``v1/core/data_engine.py``, ``v1/core/utils/batching.py``, ``v1/core/base_trainer.py``,
``v1/plugins/trainer_plugins/distributed/fsdp2.py``); sharding is done by this package's ZeRO engines
(``train/optimizer.py``, ``train/zero3.py``) instead of FSDP2."""
from .batching import BatchGenerator, StatefulBuffer  # noqa: F401
from .data_engine import DataEngine  # noqa: F401
from .model_engine import InitPlugin, KernelPlugin, ModelEngine, PeftPlugin, register_kernel  # noqa: F401
from .plugin import BatchingStrategy, DataConverter, Plugin  # noqa: F401
from .rendering import Renderer  # noqa: F401
from .trainer import SFTTrainerV1, V1TrainingArguments  # noqa: F401
