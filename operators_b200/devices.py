"""Device enum values of the C ABI (reference include/device.h:4-9,
operatorspy/devices.py:1-5).  This library serves DEVICE_CUDA only."""


class DeviceEnum:
    DEVICE_CPU = 0
    DEVICE_CUDA = 1
    DEVICE_BANG = 2
    DEVICE_ASCEND = 3
