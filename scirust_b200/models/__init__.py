from .sciagent import SciAgentConfig, GQADecoder  # noqa: F401
