"""Channel addresses and transports (hyperactor/src/channel.rs:331-500).
"""
import enum

from ..._native import ChannelRx, ChannelTx, channel_dial, channel_serve, parse_channel_addr  # noqa: F401


class ChannelTransport(enum.Enum):
    Tcp = "tcp"
    Unix = "unix"
    Local = "local"
    Sim = "sim"


class ChannelAddr:
    """``tcp:host:port`` / ``unix:/path`` / ``local:n`` / ``sim:...`` addresses."""

    def __init__(self, text: str):
        self.text = text
        self.parsed = parse_channel_addr(text)

    @staticmethod
    def any(transport: "ChannelTransport") -> str:
        from ..._native import channel_serve_any
        rx = channel_serve_any(transport.value)
        addr = rx.addr
        rx.close()
        return addr

    def __str__(self) -> str:
        return self.text
