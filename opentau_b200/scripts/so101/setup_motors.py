"""``opentau-so101-setup-motors``: give every servo its id and the bus baud rate, one motor connected at a time."""

import argparse

from .feetech import BAUDRATES, FeetechProtocol
from .motors_bus import SO101_MOTORS


def setup_motor(proto: FeetechProtocol, target_id: int, scan=range(0, 254)) -> int:
    """Finds the single motor on the bus and renumbers it; returns the id it had."""
    found = [i for i in scan if proto.ping(i)]
    if len(found) != 1:
        raise RuntimeError(f"expected exactly one motor on the bus, found ids {found}")
    cur = found[0]
    proto.write(cur, "Lock", 0)
    proto.write(cur, "Baud_Rate", BAUDRATES[1_000_000])
    if cur != target_id:
        proto.write(cur, "ID", target_id)
    proto.write(target_id, "Lock", 1)
    return cur


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--port", required=True)
    a = ap.parse_args(argv)
    import serial
    for name, m in reversed(list(SO101_MOTORS.items())):
        input(f"Connect ONLY the '{name}' motor and press Enter...")
        with serial.Serial(a.port, baudrate=1_000_000, timeout=0.05) as port:
            was = setup_motor(FeetechProtocol(port), m.id)
        print(f"'{name}': id {was} -> {m.id}")


if __name__ == "__main__":
    main()
