"""Model as data (``model``), batch description (``batch``), the step function and
graph decode (``engine``) and the generation loop (``generation``)."""
from .batch import BatchMeta, StepEntry  # noqa: F401
from .model import DecoderModel, ModelSpec, ScheduleEntry, StepContext  # noqa: F401
from .engine import Engine  # noqa: F401
