"""Small helpers shared by the host-side mirror of the reference (utils.py of the reference)."""
import os


def genKey(type_, stage_name=None, ax_name=None, param_name=None, var_name=None, others=None):
    """Variable names of the constraint model, in the reference's scheme (utils.py:21-39):
    ``L#`` loop extents, ``P#`` tunable parameters, ``V#`` derived variables, ``O#`` auxiliaries."""
    assert type_ in ["L", "P", "V", "O"]
    if type_ == "L":
        assert ax_name and stage_name
        return type_ + "#" + "ST:%s,AX:%s" % (stage_name, ax_name)
    if type_ == "P":
        assert param_name
        return type_ + "#" + "ST:%s,AX:%s,PA:%s" % (stage_name, ax_name, param_name)
    if type_ == "V":
        assert var_name
        return type_ + "#" + "ST:%s,AX:%s,VA:%s" % (stage_name, ax_name, var_name)
    assert others
    return type_ + "#" + "ST:%s,AX:%s,OT:%s" % (stage_name, ax_name, others)


def Code(point):
    """Sample identity: the solved variable vector joined by '_' (utils.py:306-311)."""
    assert isinstance(point, list)
    return "".join(str(x) + "_" for x in point)


def DeCode(code):
    assert isinstance(code, str)
    return [int(x) for x in code.split("_")[:-1]]


def removedot(name):
    return name.replace(".", "_") if isinstance(name, str) else name


def mkdir(name):
    if not os.path.exists(name):
        os.makedirs(name)
