"""Pipeline / ZeRO services under the reference's module name
(necklace/trainer/tndsmp.py).  All modes share one implementation, see service.py."""
from .service import *  # noqa: F401,F403
from .service import (MPSVCScheduler, MPSVCWorker, MPSVRScheduler, MPSVRWorker,  # noqa: F401
                      ILOG_I_MP_SCHEDULER, ILOG_I_MP_WORKER, ILOG_I_ZR_SCHEDULER,
                      ILOG_I_ZR_WORKER)


class MPSVCScheduler(MPSVCScheduler):  # noqa: F811
    """The scheduler of this flavour (see ``service.SVCScheduler.FLAVOUR``)."""
    FLAVOUR = "pp"


# the reference's log channel numbers of this flavour (necklace/trainer/tndsmp.py:14-26)
ILOG_I_MP_SVR_WKR = 600001
ILOG_I_MP_SVC_WKR = 600002
ILOG_I_MP_SVR_SCH = 600003
ILOG_I_MP_SVC_SCH = 600004
