// Nothing from boost/utility.hpp is used by the engine sources built here.
