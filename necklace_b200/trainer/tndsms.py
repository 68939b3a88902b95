"""Scheduler / worker services under the reference's module name
(necklace/trainer/tndsms.py).  All modes share one implementation, see service.py."""
from .service import *  # noqa: F401,F403
from .service import (SVCScheduler, SVCWorker, SVRScheduler, SVRWorker,  # noqa: F401
                      ILOG_I_SVC_SCHEDULER, ILOG_I_SVC_WORKER)
