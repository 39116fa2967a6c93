from .dpscheduler import DPScheduler, DPSchedulerMax, DPSChedulerRR, get_dp_scheduler  # noqa: F401
