"""dynaflow_b200: B200-native execution backend behind DynaFlow's scheduling API."""
__version__ = "0.1.0"
