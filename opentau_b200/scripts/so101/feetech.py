"""Feetech STS/SMS serial protocol and the STS3215 control table
(reference ``src/opentau/scripts/so101/motors/feetech/{feetech,tables}.py``).

Packet: ``FF FF id len instr params... checksum`` with ``checksum = ~(id + len + instr + sum(params)) & 0xFF`` and
``len = len(params) + 2``; multi-byte registers are little endian; negative values use sign-magnitude with the sign in
a model-specific bit.  The transport is any object with ``write(bytes)``, ``read(n) -> bytes`` and ``reset_input_buffer()``
(``serial.Serial`` on a real bus, :class:`FakeFeetechPort` in tests).
"""

from __future__ import annotations

PING, READ, WRITE, REG_WRITE, ACTION, SYNC_READ, SYNC_WRITE = 0x01, 0x02, 0x03, 0x04, 0x05, 0x82, 0x83
BROADCAST_ID = 0xFE

# name -> (address, size in bytes)
STS3215_TABLE: dict[str, tuple[int, int]] = {
    "Model_Number": (3, 2), "ID": (5, 1), "Baud_Rate": (6, 1), "Return_Delay_Time": (7, 1),
    "Min_Position_Limit": (9, 2), "Max_Position_Limit": (11, 2), "Max_Torque_Limit": (16, 2), "P_Coefficient": (21, 1),
    "D_Coefficient": (22, 1), "I_Coefficient": (23, 1), "Homing_Offset": (31, 2), "Operating_Mode": (33, 1),
    "Torque_Enable": (40, 1), "Acceleration": (41, 1), "Goal_Position": (42, 2), "Goal_Velocity": (46, 2),
    "Torque_Limit": (48, 2), "Lock": (55, 1), "Present_Position": (56, 2), "Present_Velocity": (58, 2),
    "Present_Load": (60, 2), "Present_Voltage": (62, 1), "Present_Temperature": (63, 1), "Moving": (66, 1),
    "Present_Current": (69, 2), "Maximum_Acceleration": (85, 1),
}
SIGN_BIT = {"Homing_Offset": 11, "Goal_Velocity": 15, "Present_Velocity": 15, "Present_Load": 10, "Present_Current": 15}
BAUDRATES = {1_000_000: 0, 500_000: 1, 250_000: 2, 128_000: 3, 115_200: 4, 57_600: 5, 38_400: 6, 19_200: 7}
RESOLUTION = 4096


class FeetechError(IOError):
    pass


def checksum(body: bytes) -> int:
    return (~sum(body)) & 0xFF


def build_packet(motor_id: int, instr: int, params: bytes = b"") -> bytes:
    body = bytes([motor_id, len(params) + 2, instr]) + params
    return b"\xff\xff" + body + bytes([checksum(body)])


def encode_sign(name: str, value: int) -> int:
    bit = SIGN_BIT.get(name)
    if bit is None:
        return value
    mag = abs(value)
    if mag >= (1 << bit):
        raise ValueError(f"{name}={value} does not fit {bit} magnitude bits")
    return mag | ((1 << bit) if value < 0 else 0)


def decode_sign(name: str, raw: int) -> int:
    bit = SIGN_BIT.get(name)
    if bit is None:
        return raw
    mag = raw & ((1 << bit) - 1)
    return -mag if raw & (1 << bit) else mag


def to_bytes(value: int, size: int) -> bytes:
    return int(value).to_bytes(size, "little", signed=False)


class FeetechProtocol:
    def __init__(self, port, timeout_reads: int = 3):
        self.port, self.retries = port, timeout_reads

    # -- low level ------------------------------------------------------------------------------------
    def _read_status(self, expect_id: int) -> bytes:
        hdr = self.port.read(4)
        if len(hdr) < 4 or hdr[:2] != b"\xff\xff":
            raise FeetechError(f"no / bad status header from motor {expect_id}: {hdr.hex()}")
        mid, length = hdr[2], hdr[3]
        rest = self.port.read(length)
        if len(rest) < length:
            raise FeetechError(f"truncated status packet from motor {mid}")
        err, params, chk = rest[0], rest[1:-1], rest[-1]
        if checksum(bytes([mid, length]) + rest[:-1]) != chk:
            raise FeetechError(f"checksum mismatch in the status packet of motor {mid}")
        if mid != expect_id:
            raise FeetechError(f"status packet from motor {mid}, expected {expect_id}")
        if err & ~0x20:            # bit 5 = overload warning only
            raise FeetechError(f"motor {mid} reports error flags 0x{err:02x}")
        return params

    def _txrx(self, motor_id: int, instr: int, params: bytes) -> bytes:
        last: Exception | None = None
        for _ in range(self.retries):
            self.port.reset_input_buffer()
            self.port.write(build_packet(motor_id, instr, params))
            try:
                return self._read_status(motor_id)
            except FeetechError as e:
                last = e
        raise last  # type: ignore[misc]

    # -- instructions -----------------------------------------------------------------------------------
    def ping(self, motor_id: int) -> bool:
        try:
            self._txrx(motor_id, PING, b"")
            return True
        except FeetechError:
            return False

    def read(self, motor_id: int, name: str) -> int:
        addr, size = STS3215_TABLE[name]
        data = self._txrx(motor_id, READ, bytes([addr, size]))
        if len(data) != size:
            raise FeetechError(f"motor {motor_id}: read of {name} returned {len(data)} bytes, expected {size}")
        return decode_sign(name, int.from_bytes(data, "little"))

    def write(self, motor_id: int, name: str, value: int) -> None:
        addr, size = STS3215_TABLE[name]
        self._txrx(motor_id, WRITE, bytes([addr]) + to_bytes(encode_sign(name, value), size))

    def sync_write(self, name: str, values: dict[int, int]) -> None:
        addr, size = STS3215_TABLE[name]
        params = bytes([addr, size])
        for mid, v in values.items():
            params += bytes([mid]) + to_bytes(encode_sign(name, v), size)
        self.port.write(build_packet(BROADCAST_ID, SYNC_WRITE, params))        # no status packet for broadcasts

    def sync_read(self, name: str, ids: list[int]) -> dict[int, int]:
        addr, size = STS3215_TABLE[name]
        self.port.reset_input_buffer()
        self.port.write(build_packet(BROADCAST_ID, SYNC_READ, bytes([addr, size]) + bytes(ids)))
        out = {}
        for mid in ids:
            data = self._read_status(mid)
            out[mid] = decode_sign(name, int.from_bytes(data, "little"))
        return out


class FakeFeetechPort:
    """In-memory bus of STS3215 servos for tests and dry runs: registers per motor, answers READ / WRITE / PING /
    SYNC_READ / SYNC_WRITE; ``Present_Position`` follows ``Goal_Position`` while torque is on."""

    def __init__(self, ids: list[int]):
        self.regs = {i: bytearray(128) for i in ids}
        for i in ids:
            self._set(i, "ID", i)
            self._set(i, "Model_Number", 777)
            self._set(i, "Present_Position", 2048)
            self._set(i, "Goal_Position", 2048)
            self._set(i, "Max_Position_Limit", 4095)
            self._set(i, "Present_Voltage", 120)
            self._set(i, "Present_Temperature", 30)
        self.rx = bytearray()
        self.writes: list[bytes] = []

    def _set(self, i: int, name: str, v: int) -> None:
        a, s = STS3215_TABLE[name]
        self.regs[i][a:a + s] = to_bytes(v, s)

    def _get(self, i: int, name: str) -> int:
        a, s = STS3215_TABLE[name]
        return int.from_bytes(self.regs[i][a:a + s], "little")

    def reset_input_buffer(self) -> None:
        self.rx.clear()

    def read(self, n: int) -> bytes:
        out, self.rx = bytes(self.rx[:n]), self.rx[n:]
        return out

    def _status(self, mid: int, params: bytes = b"") -> None:
        body = bytes([mid, len(params) + 2, 0]) + params
        self.rx += b"\xff\xff" + body + bytes([checksum(body)])

    def _apply_write(self, mid: int, addr: int, data: bytes) -> None:
        if mid not in self.regs:
            return
        self.regs[mid][addr:addr + len(data)] = data
        ga, gs = STS3215_TABLE["Goal_Position"]
        if addr <= ga < addr + len(data) and self._get(mid, "Torque_Enable"):
            self._set(mid, "Present_Position", self._get(mid, "Goal_Position"))
        ia, _ = STS3215_TABLE["ID"]
        if addr == ia and data[0] != mid:                       # the motor answers under its new id from now on
            self.regs[data[0]] = self.regs.pop(mid)

    def write(self, pkt: bytes) -> int:
        self.writes.append(bytes(pkt))
        if pkt[:2] != b"\xff\xff" or checksum(pkt[2:-1]) != pkt[-1]:
            return len(pkt)
        mid, instr, params = pkt[2], pkt[4], pkt[5:-1]
        if instr == PING and mid in self.regs:
            self._status(mid)
        elif instr == READ and mid in self.regs:
            self._status(mid, bytes(self.regs[mid][params[0]:params[0] + params[1]]))
        elif instr == WRITE and mid in self.regs:
            self._status(mid)                                   # the acknowledgement still carries the old id
            self._apply_write(mid, params[0], params[1:])
        elif instr == SYNC_WRITE:
            addr, size = params[0], params[1]
            for k in range(2, len(params), size + 1):
                self._apply_write(params[k], addr, params[k + 1:k + 1 + size])
        elif instr == SYNC_READ:
            addr, size = params[0], params[1]
            for m in params[2:]:
                if m in self.regs:
                    self._status(m, bytes(self.regs[m][addr:addr + size]))
        return len(pkt)

    def close(self) -> None:
        pass
