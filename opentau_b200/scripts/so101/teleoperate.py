"""``opentau-so101-teleoperate``: the follower mirrors the leader at a fixed rate."""

import argparse
import time

from .devices import SOArmConfig, SOFollower, SOLeader, busy_wait, teleoperate_step


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--leader-port", required=True)
    ap.add_argument("--follower-port", required=True)
    ap.add_argument("--fps", type=int, default=60)
    ap.add_argument("--duration", type=float, default=None)
    a = ap.parse_args(argv)
    leader, follower = SOLeader(SOArmConfig(port=a.leader_port, id="leader")), SOFollower(SOArmConfig(port=a.follower_port, id="follower"))
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
