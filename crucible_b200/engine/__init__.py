from .context import CacheStorage, HostStep, Scratch, StepContext, StepLayout
from .engine import DEVICE_TOKEN, Engine, EngineOptions, StepEntry, StepError, parse_dtype
