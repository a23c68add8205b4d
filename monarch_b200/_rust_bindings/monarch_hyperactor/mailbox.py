"""Mailboxes and ports (monarch_hyperactor/src/mailbox.rs:68-755).
"""
from ..._native import AccumReceiver, Envelope, Instance as Mailbox, QueueReceiver, parse_port_id  # noqa: F401
from ...actor.actor_mesh import Accumulator, Port, PortReceiver  # noqa: F401

PortHandle = PortRef = OncePortHandle = OncePortRef = Port
OncePortReceiver = PortReceiverBase = PortReceiver
UndeliverablePortReceiver = QueueReceiver
UndeliverableMessageEnvelope = Envelope


class PortId:
    """``world[rank].actor[pid][port]`` (hyperactor/src/reference.rs:332-400)."""

    def __init__(self, text: str):
        self.text = text
        self.actor_id, self.port = parse_port_id(text)

    @staticmethod
    def from_string(text: str) -> "PortId":
        return PortId(text)

    def __str__(self) -> str:
        return self.text


class Reducer:
    """Names of the reducers folded natively in mailboxes and along cast trees."""
    SUM_F32, SUM_F64, MAX_F64, MIN_F64, SUM_I64 = "sum_f32", "sum_f64", "max_f64", "min_f64", "sum_i64"
