"""``python -m torchft_b200.lighthouse_cli --min_replicas N [--bind [::]:29510] ...``

Stand-alone lighthouse (quorum service + dashboard at ``http://host:port/``).  Flags:
``--bind``, ``--min_replicas`` (required), ``--join_timeout_ms`` (60000),
``--quorum_tick_ms`` (100), ``--heartbeat_timeout_ms`` (5000).  Equivalent of the
reference's ``torchft_lighthouse`` console script (src/bin/lighthouse.rs:11-24)."""

import sys

from ._ftcp import lighthouse_main


def main() -> None:
    sys.exit(lighthouse_main(["torchft_b200_lighthouse"] + sys.argv[1:]))


if __name__ == "__main__":
    main()
