from .task import KernelHandle, Task
