"""Decisions shared by runner jobs (reference: axlearn/cloud/gcp/runners/utils.py:10-60)."""

from __future__ import annotations

import logging
from typing import Optional

# Processor types whose capacity comes either from a reservation (scheduling tier 0) or from spot
# nodes (other tiers).  The reference only recreates TPU jobs; GPU node pools have the same two
# sources here.
RESCHEDULABLE_PROCESSORS = ("gpu", "tpu")


def should_recreate_job(tier: Optional[str], reservation: Optional[str], processor_type: Optional[str],
                        is_pending: bool = False) -> bool:
    """Whether a job that the scheduler put on ``tier`` while its resources use ``reservation``
    should be torn down and created again.

    * tier other than 0 (and not "disabled") but holding a reservation: recreate, the reservation
      belongs to tier-0 jobs;
    * tier 0 without a reservation: recreate only while the job is pending -- a running job keeps its
      spot nodes until it is pre-empted, so that jobs bouncing between tiers are not restarted over
      and over;
    * an unknown processor type never recreates.
    """
    if processor_type not in RESCHEDULABLE_PROCESSORS:
        return False
    if str(tier) not in ("0", "disabled") and reservation is not None:
        logging.info("Bastion tier is %s but reservation is %s. Job resources will be recreated.", tier, reservation)
        return True
    if str(tier) == "0" and reservation is None:
        if is_pending:
            logging.info("Bastion tier is %s but there is no reservation; the job is pending, recreating it.", tier)
            return True
        logging.info("Bastion tier is %s but there is no reservation; the job is active and runs until pre-emption.", tier)
    return False
