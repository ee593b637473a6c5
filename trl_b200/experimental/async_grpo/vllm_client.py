"""Generation-server client used by the async worker (trl/experimental/async_grpo/vllm_client.py:20-100): the stable
client already speaks the server's routes, including weight pushes."""
from ...generation.client import VLLMClient

__all__ = ["VLLMClient"]
