from rl_engine.utils.logger import init_logger, logger

__all__ = ["init_logger", "logger"]
