"""Runtime services around the kernels: measured tuning decisions kept per device."""
from .tuning import Tuner, device_key, reset_tuner, size_class, tuner
