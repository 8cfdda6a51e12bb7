from .codebook import LloydMaxCalibrator, calibrate_codebook, calibrate_per_group
from .qjl import RademacherQJL, qjl_encode, qjl_reconstruct

__all__ = ["LloydMaxCalibrator", "calibrate_codebook", "calibrate_per_group",
           "RademacherQJL", "qjl_encode", "qjl_reconstruct"]
