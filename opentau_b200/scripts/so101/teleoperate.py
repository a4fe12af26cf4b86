"""``opentau-so101-teleoperate``: the follower mirrors the leader at a fixed rate."""

import argparse
import time

from .devices import (BiSOArmConfig, BiSOFollower, BiSOLeader, SOArmConfig, SOFollower, SOLeader, busy_wait,
                      teleoperate_step)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--leader-port", required=True)
    ap.add_argument("--follower-port", required=True)
    ap.add_argument("--leader-port-right", default=None, help="bimanual: the right leader arm (the first is the left)")
    ap.add_argument("--follower-port-right", default=None, help="bimanual: the right follower arm")
    ap.add_argument("--fps", type=int, default=60)
    ap.add_argument("--duration", type=float, default=None)
    a = ap.parse_args(argv)
    if (a.leader_port_right is None) != (a.follower_port_right is None):
        ap.error("bimanual teleoperation needs both --leader-port-right and --follower-port-right")
    if a.leader_port_right:
        leader = BiSOLeader(BiSOArmConfig(SOArmConfig(port=a.leader_port), SOArmConfig(port=a.leader_port_right),
                                          id="leader"))
        follower = BiSOFollower(BiSOArmConfig(SOArmConfig(port=a.follower_port),
                                              SOArmConfig(port=a.follower_port_right), id="follower"))
    else:
        leader = SOLeader(SOArmConfig(port=a.leader_port, id="leader"))
        follower = SOFollower(SOArmConfig(port=a.follower_port, id="follower"))
    leader.connect()
    follower.connect()
    t_end = None if a.duration is None else time.perf_counter() + a.duration
    try:
        while t_end is None or time.perf_counter() < t_end:
            t0 = time.perf_counter()
            teleoperate_step(leader, follower)
            busy_wait(max(0.0, 1 / a.fps - (time.perf_counter() - t0)))
    finally:
        leader.disconnect()
        follower.disconnect()


if __name__ == "__main__":
    main()
