"""Pipeline / ZeRO services under the reference's module name
(necklace/trainer/tndspp.py).  All modes share one implementation, see service.py."""
from .service import *  # noqa: F401,F403
from .service import (MPSVCScheduler, MPSVCWorker, MPSVRScheduler, MPSVRWorker,  # noqa: F401
                      ILOG_I_MP_SCHEDULER, ILOG_I_MP_WORKER, ILOG_I_ZR_SCHEDULER,
                      ILOG_I_ZR_WORKER)


class MPSVCScheduler(MPSVCScheduler):  # noqa: F811
    """The scheduler of this flavour (see ``service.SVCScheduler.FLAVOUR``)."""
    FLAVOUR = "pp"


# the reference's log channel numbers of this flavour (necklace/trainer/tndspp.py:14-26)
ILOG_I_MP_SVR_WKR = 600011
ILOG_I_MP_SVR_WKR_PRT = 600015
ILOG_I_MP_SVC_WKR = 600012
ILOG_I_MP_SVC_WKR_PRT = 600016
ILOG_I_MP_SVR_SCH = 600021
ILOG_I_MP_SVR_SCH_PRT = 600025
ILOG_I_MP_SVC_SCH = 600022
ILOG_I_MP_SVC_SCH_PRT = 600026
