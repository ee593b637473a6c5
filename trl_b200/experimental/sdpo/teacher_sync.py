"""Teacher maintenance for SDPO: the same base / ema / student choices as SDFT (``experimental/sdft/teacher_sync.py``)."""
from ..sdft.teacher_sync import TeacherSyncCallback, build_teacher  # noqa: F401
