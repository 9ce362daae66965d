from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, expected_weights

__all__ = ["LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "expected_weights"]
