"""Pipeline / ZeRO services under the reference's module name
(necklace/trainer/tndszr.py).  All modes share one implementation, see service.py."""
from .service import *  # noqa: F401,F403
from .service import (MPSVCScheduler, MPSVCWorker, MPSVRScheduler, MPSVRWorker,  # noqa: F401
                      ILOG_I_MP_SCHEDULER, ILOG_I_MP_WORKER, ILOG_I_ZR_SCHEDULER,
                      ILOG_I_ZR_WORKER)
